// Input transform V = B^T d B fused with the gather from NCHW / NHWC / CHWN.
//
// Replaces wino_input_trans_nchw_suitFor128_2 / _nhwc_suitFor128 / _chwn_suitFor128
// (comparison/wrapedConv_NCHW.cuh:760-856, wrapedConv_NHWC.cuh:266-329, wrapedConv_CHWN.cuh:225-275),
// which map one thread to one (tile, channel) and issue a*a scalar stores at plane stride.
//
// Every layout writes the same operand buffer V[xi][tile][Cp] (channels contiguous = the K-major operand the
// tile GEMM wants), so the layouts differ only in how a CTA stages its input patch in shared memory.  The
// staged patch is an array of 128-byte rows, one row per spatial position, holding 32 4-byte "words" of
// channel data (two bf16 channels or one float channel per word).  The transform step is the same everywhere:
// warp w owns tile w of the unit, lane l owns word l; shared-memory reads are conflict free and every global
// store instruction writes one full 128-byte line of V.
//   * NHWC, pixel pitch a multiple of 16 bytes: persistent CTAs, the a x (8m+2) x 128-byte halo patch of 8
//     adjacent tiles arrives by ONE 4-D cp.async.bulk.tensor load into a 3-deep ring; rows, columns and channels
//     outside the tensor are zero filled by the TMA unit (= the zero padding and the Cp padding of V);
//   * NCHW: the same unit, loaded with 16-byte vectors along w (aligned chunks that cover the halo row) and
//     scattered into the word rows; lanes run along channels so the scatter is conflict free;
//   * CHWN: unit = one tile position x 8 images x 128 bytes of channels, loaded with 16-byte vectors along n;
//   * NCHW and CHWN with 16-byte-aligned rows (every float case of the VGG shapes, bf16 NCHW with W a multiple of 8, bf16
//     CHWN with N a multiple of 8): the same units, but the patch of channel planes arrives as one TMA box in
//     persistent CTAs and is turned around inside shared memory (input_transform_planar_tma);
//   * NHWC with an unaligned pixel pitch (C = 3, 20, ...): scalar loads, lanes along channels.
// HBM bound: reads N*C*H*W elements (x ~1.5 through L2 for the vertical halo), writes a*a*T*Cp.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "wino_math.cuh"

namespace wino {

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

constexpr int IT_TX = 8;    // tiles per unit along x (NHWC, NCHW)
constexpr int IT_NB = 8;    // images per unit (CHWN)

// ---- word <-> float conversion ------------------------------------------------------------------------
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

// Transforms the a x a patch whose words sit at src[(r*row_stride + s*col_stride) * PITCH] and stores the a*a
// results as words at dst[xi * plane_words].
// SWZ: the word of lane l for patch element (r, q) sits at column l ^ (r*A + q) of its row (CHWN staging).
template <int A, typename TIn, typename TOp, bool SWZ = false, int PITCH = 32>
__device__ __forceinline__ void transform_words(const uint32_t* src, int row_stride, int col_stride, uint32_t* dst,
                                                long long plane_words, int lane = 0) {
    using IO = WordIO<TIn, TOp>;
    uint32_t w[A][A];
#pragma unroll
    for (int r = 0; r < A; ++r)
#pragma unroll
        for (int q = 0; q < A; ++q)
            w[r][q] = src[(r * row_stride + q * col_stride) * PITCH + (SWZ ? (lane ^ ((r * A + q) & 31)) : 0)];
    if constexpr (IO::VEC == 2) {
        // two channels per word: both go through the transform together as packed FP32 pairs
        vf2 d[A][A], o[A][A];
#pragma unroll
        for (int r = 0; r < A; ++r)
#pragma unroll
            for (int q = 0; q < A; ++q) d[r][q].v = make_float2(IO::get(w[r][q], 0), IO::get(w[r][q], 1));
        input_tile_transform<A, vf2>(d, o);
#pragma unroll
        for (int r = 0; r < A; ++r)
#pragma unroll
            for (int q = 0; q < A; ++q) dst[(long long)(r * A + q) * plane_words] = IO::put(o[r][q].v.x, o[r][q].v.y);
    } else {
        vf1 d[A][A], o[A][A];
#pragma unroll
        for (int r = 0; r < A; ++r)
#pragma unroll
            for (int q = 0; q < A; ++q) d[r][q].v = IO::get(w[r][q], 0);
        input_tile_transform<A, vf1>(d, o);
#pragma unroll
        for (int r = 0; r < A; ++r)
#pragma unroll
            for (int q = 0; q < A; ++q) dst[(long long)(r * A + q) * plane_words] = IO::put(o[r][q].v, 0.f);
    }
}

// writes element (channel c_l of the unit) of spatial position `pos` into the staged word rows
template <typename TIn>
__device__ __forceinline__ void put_element(uint8_t* patch, int pos, int c_l, TIn v) {
    reinterpret_cast<TIn*>(patch + pos * 128)[c_l] = v;
}

// ---- NHWC (unaligned pitch), NCHW: strip unit, cooperative loads ---------------------------------------
template <int A, bool NCHW_IN, typename TIn, typename TOp>
__global__ void __launch_bounds__(256, 3) input_transform_strip(const ITArgs a, const int bxchunks, const int cchunks) {
    constexpr int M = A - 2;
    constexpr int COLS = M * IT_TX + 2;
    constexpr int VEC = 4 / (int)sizeof(TIn);
    constexpr int CH = 32 * VEC;                   // channels per unit
    constexpr int VE = 16 / (int)sizeof(TIn);      // elements per 16-byte vector
    __shared__ __align__(16) uint8_t patch[A * COLS * 128];

    const int c0 = (blockIdx.x % cchunks) * CH;
    const int bx0 = (blockIdx.x / cchunks) * IT_TX;
    const int by = blockIdx.y;
    const int n = a.n0 + blockIdx.z;
    const int gh0 = by * M - a.pad, gw0 = bx0 * M - a.pad;
    const TIn* __restrict__ x = reinterpret_cast<const TIn*>(a.x) + (long long)n * a.sx.n;
    const TIn zero = from_float<TIn>(0.f);

    if (NCHW_IN) {
        // aligned 16-byte chunks along w that cover columns [gw0, gw0 + COLS); lanes run along channels
        const int ws = (gw0 >= 0 ? gw0 / VE : -((-gw0 + VE - 1) / VE)) * VE;
        const int off = gw0 - ws;                                  // 0 .. VE-1
        const int nchunks = (off + COLS + VE - 1) / VE;
        const bool vec_ok = (a.W % VE) == 0 && ((a.sx.n | a.sx.c) % VE) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;
        // two phases, fully unrolled: every load of the thread is in flight before the first scatter into shared memory
        // (a single loop makes each load wait for the one before it, one DRAM latency per pass)
        constexpr int MAXCHUNKS = (COLS + 2 * (VE - 1) + VE - 1) / VE;
        constexpr int PASSES = (CH * A * MAXCHUNKS + 255) / 256;
        const int items = CH * A * nchunks;
        uint4 held[PASSES];
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const int item = threadIdx.x + 256 * i;
            if (item >= items) continue;
            const int c_l = item % CH;
            const int rc = item / CH;
            const int r = rc % A, chunk = rc / A;
            const int gh = gh0 + r, gw = ws + chunk * VE, c = c0 + c_l;
            __align__(16) TIn vals[VE];
            const bool row_ok = gh >= 0 && gh < a.H && c < a.C;
            if (row_ok && vec_ok && gw >= 0 && gw + VE <= a.W) {
                *reinterpret_cast<uint4*>(vals) = *reinterpret_cast<const uint4*>(x + c * a.sx.c + gh * a.sx.h + gw);
            } else {
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    const int w = gw + e;
                    vals[e] = (row_ok && w >= 0 && w < a.W) ? x[c * a.sx.c + gh * a.sx.h + w] : zero;
                }
            }
            held[i] = *reinterpret_cast<const uint4*>(vals);
        }
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
            const int item = threadIdx.x + 256 * i;
            if (item >= items) continue;
            const int c_l = item % CH;
            const int rc = item / CH;
            const int r = rc % A, chunk = rc / A;
            __align__(16) TIn vals[VE];
            *reinterpret_cast<uint4*>(vals) = held[i];
#pragma unroll
            for (int e = 0; e < VE; ++e) {
                const int col = chunk * VE + e - off;
                if (col >= 0 && col < COLS) put_element<TIn>(patch, r * COLS + col, c_l, vals[e]);
            }
        }
    } else {
        for (int item = threadIdx.x; item < A * COLS * CH; item += 256) {
            const int c_l = item % CH;
            const int rc = item / CH;
            const int col = rc % COLS, r = rc / COLS;
            const int gh = gh0 + r, gw = gw0 + col, c = c0 + c_l;
            TIn val = zero;
            if (gh >= 0 && gh < a.H && gw >= 0 && gw < a.W && c < a.C) val = x[c * a.sx.c + gh * a.sx.h + gw * a.sx.w];
            put_element<TIn>(patch, r * COLS + col, c_l, val);
        }
    }
    __syncthreads();

    const int tl = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int bx = bx0 + tl, c = c0 + lane * VEC;
    if (bx < a.bnx && c < a.cp) {
        const long long t = ((long long)blockIdx.z * a.bny + by) * a.bnx + bx;
        transform_words<A, TIn, TOp>(reinterpret_cast<const uint32_t*>(patch) + (tl * M) * 32 + lane, COLS, 1,
                                     reinterpret_cast<uint32_t*>(a.v) + (t * a.cp + c) / VEC, a.tp * a.cp / VEC);
    }
}

// ---- CHWN: batch unit (one tile position, 8 images), 16-byte loads along n ---------------------------------
template <int A, typename TIn, typename TOp>
__global__ void __launch_bounds__(256, 3) input_transform_batch(const ITArgs a, const int cchunks) {
    constexpr int M = A - 2;
    constexpr int VEC = 4 / (int)sizeof(TIn);
    constexpr int CH = 32 * VEC;
    constexpr int VE = 16 / (int)sizeof(TIn);      // images per 16-byte vector: 8 (bf16) or 4 (float)
    constexpr int NV = IT_NB / VE;                 // vectors per 8 images
    __shared__ __align__(16) uint8_t patch[A * A * IT_NB * 128];

    const int c0 = (blockIdx.x % cchunks) * CH;
    const int nb0 = (blockIdx.x / cchunks) * IT_NB;
    const int bx = blockIdx.y, by = blockIdx.z;
    const int gh0 = by * M - a.pad, gw0 = bx * M - a.pad;
    const TIn* __restrict__ x = reinterpret_cast<const TIn*>(a.x);
    const TIn zero = from_float<TIn>(0.f);
    const int nbase = a.n0 + nb0;
    // sx.n == 1: images are contiguous; a vector of VE images is aligned when every stride and the base are
    const bool vec_ok = ((a.sx.c | a.sx.h | a.sx.w) % VE) == 0 && (nbase % VE) == 0 && (reinterpret_cast<uintptr_t>(a.x) & 15) == 0;

    // lanes run over the a*a patch positions of ONE channel (addresses inside one channel plane); the word column
    // is XOR-swizzled with the position so that this scatter and the transform's reads are both conflict free
    // two phases, fully unrolled: all of the thread's loads are in flight before the first scatter
    constexpr int PASSES = (CH * A * A * NV + 255) / 256;
    uint4 held[PASSES];
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
        const int item = threadIdx.x + 256 * i;
        if (item >= CH * A * A * NV) continue;
        const int rs = item % (A * A);
        const int rc = item / (A * A);
        const int nv = rc % NV, c_l = rc / NV;
        const int gh = gh0 + rs / A, gw = gw0 + rs % A, c = c0 + c_l;
        const int n_l0 = nv * VE;
        __align__(16) TIn vals[VE];
        const bool ok = gh >= 0 && gh < a.H && gw >= 0 && gw < a.W && c < a.C;
        const TIn* src = x + c * a.sx.c + gh * a.sx.h + gw * a.sx.w + (nbase + n_l0);
        if (ok && vec_ok && nb0 + n_l0 + VE <= a.ns) {
            *reinterpret_cast<uint4*>(vals) = *reinterpret_cast<const uint4*>(src);
        } else {
#pragma unroll
            for (int e = 0; e < VE; ++e) vals[e] = (ok && nb0 + n_l0 + e < a.ns) ? src[e] : zero;
        }
        held[i] = *reinterpret_cast<const uint4*>(vals);
    }
#pragma unroll
    for (int i = 0; i < PASSES; ++i) {
        const int item = threadIdx.x + 256 * i;
        if (item >= CH * A * A * NV) continue;
        const int rs = item % (A * A);
        const int rc = item / (A * A);
        const int nv = rc % NV, c_l = rc / NV;
        const int n_l0 = nv * VE;
        __align__(16) TIn vals[VE];
        *reinterpret_cast<uint4*>(vals) = held[i];
        const int word = (c_l / VEC) ^ (rs & 31);
#pragma unroll
        for (int e = 0; e < VE; ++e) put_element<TIn>(patch, rs * IT_NB + n_l0 + e, word * VEC + (c_l % VEC), vals[e]);
    }
    __syncthreads();

    const int n_l = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int c = c0 + lane * VEC;
    if (nb0 + n_l < a.ns && c < a.cp) {
        const long long t = ((long long)(nb0 + n_l) * a.bny + by) * a.bnx + bx;
        transform_words<A, TIn, TOp, true>(reinterpret_cast<const uint32_t*>(patch) + n_l * 32, A * IT_NB, IT_NB,
                                           reinterpret_cast<uint32_t*>(a.v) + (t * a.cp + c) / VEC, a.tp * a.cp / VEC, lane);
    }
}

// ---- NCHW / CHWN whose rows the TMA unit can address: channel planes staged by TMA, turned around in shared memory ----
// The two kernels above stage a unit through registers and spend as many instructions on the gather as on the
// transform; on B200 they reach 0.41 - 0.49 of the HBM copy rate, limited by instruction latency.  Where every stride of
// x is a multiple of 16 bytes the gather is handed to the TMA unit:
//   * ONE 4-D box per unit brings the patch of 128 bytes' worth of channels in (32 float or 64 bf16 channels),
//     channel-major as it lies in memory (NCHW: planes of A rows x BOXW columns starting on a 16-byte boundary at or left
//     of the patch; CHWN: planes of A x A pixels x 8 images); rows, columns, channels and images outside the tensor
//     arrive as zeros (= the padding of the convolution and of V).  The box of the unit after the next is in flight
//     while a unit is processed (ring of two);
//   * the CTA turns the box around inside shared memory into the [position][word of channels] rows the transform step
//     reads (pitch 33 words: the writes, lanes along positions, and the reads, lanes along channels, are both conflict
//     free; two bf16 channel planes are zipped into one word on the way);
//   * transform and store as above.
constexpr int ITP_WAIT_CODE = 6;

template <int A, bool CHWN_IN, typename TIn>
struct PlanarUnit {
    static constexpr int ES = (int)sizeof(TIn);
    static constexpr int VEC = 4 / ES;                                      // channels per word
    static constexpr int EPV = 16 / ES;                                     // elements per 16 bytes
    static constexpr int M = A - 2;
    static constexpr int COLS = M * IT_TX + 2;                              // NCHW: patch columns of 8 adjacent tiles
    static constexpr int BOXW = (COLS + EPV - 1 + EPV - 1) / EPV * EPV;     // ... covered from a 16-byte boundary
    static constexpr int POS = CHWN_IN ? A * A * IT_NB : A * COLS;          // positions the transform reads
    static constexpr int RAW = CHWN_IN ? A * A * IT_NB : A * BOXW;          // elements per channel in the box
    static constexpr int CH = 32 * VEC;                                     // channels per unit
    static constexpr int STAGES = 2;
    static constexpr int STAGE_BYTES = CH * RAW * ES;                       // a multiple of 128
    static constexpr int TPITCH = 33;
    static constexpr int TBUF_BYTES = (POS * TPITCH * 4 + 127) / 128 * 128;
    static constexpr int SMEM = STAGES * STAGE_BYTES + TBUF_BYTES + 8 * STAGES + 16;
    static constexpr int PER_LANE = (POS + 31) / 32;                        // positions per lane and word in the turn-around
};

template <int A, bool CHWN_IN, typename TIn, typename TOp>
__global__ void __launch_bounds__(256, 2)
input_transform_planar_tma(const __grid_constant__ CUtensorMap tm_x, const ITArgs a, const int xchunks, const int cchunks,
                           const long long units, int* status) {
    using U = PlanarUnit<A, CHWN_IN, TIn>;
    constexpr int M = U::M, COLS = U::COLS, BOXW = U::BOXW, CH = U::CH, STAGES = U::STAGES, TP = U::TPITCH, VEC = U::VEC, EPV = U::EPV;
    extern __shared__ __align__(1024) uint8_t smem_planar[];
    const uint32_t ring = smem_u32(smem_planar);
    uint32_t* tbuf = reinterpret_cast<uint32_t*>(smem_planar + STAGES * U::STAGE_BYTES);
    const uint32_t bars = ring + STAGES * U::STAGE_BYTES + U::TBUF_BYTES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_planar + STAGES * U::STAGE_BYTES + U::TBUF_BYTES + 8 * STAGES);

    const long long first = blockIdx.x;
    const long long n_my = first < units ? (units - first + gridDim.x - 1) / gridDim.x : 0;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_init(bars + 8 * s, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();

    // unit -> (channel chunk, x chunk, q, z); the channel chunk runs fastest so that CTAs working side by side write
    // neighbouring 128-byte pieces of the same V rows
    //   NCHW: xchunks = chunks of 8 tiles along x;   q = tile row by,    z = image of the slab
    //   CHWN: xchunks = chunks of 8 images;          q = tile column bx, z = tile row by
    auto decode = [&](long long i, int& c0, int& xc, int& q, int& z) {
        long long u = first + i * gridDim.x;
        c0 = (int)(u % cchunks) * CH; u /= cchunks;
        xc = (int)(u % xchunks); u /= xchunks;
        const int qn = CHWN_IN ? a.bnx : a.bny;
        q = (int)(u % qn);
        z = (int)(u / qn);
    };
    // first patch column of an NCHW unit rounded down to a 16-byte boundary of the row
    auto box_start = [&](int xc) {
        const int gw0 = xc * IT_TX * M - a.pad;
        return gw0 >= 0 ? gw0 / EPV * EPV : -((-gw0 + EPV - 1) / EPV * EPV);
    };
    auto issue = [&](long long i) {          // one thread
        int c0, xc, q, z;
        decode(i, c0, xc, q, z);
        const int s = (int)(i % STAGES);
        mbar_arrive_expect_tx(bars + 8 * s, U::STAGE_BYTES);
        if (CHWN_IN) tma_load_4d(ring + s * U::STAGE_BYTES, &tm_x, bars + 8 * s, a.n0 + xc * IT_NB, q * M - a.pad, z * M - a.pad, c0);
        else tma_load_4d(ring + s * U::STAGE_BYTES, &tm_x, bars + 8 * s, box_start(xc), q * M - a.pad, c0, a.n0 + z);
    };
    if (threadIdx.x == 0)
        for (long long i = 0; i < n_my && i < STAGES; ++i) issue(i);

    const int wv = threadIdx.x / 32, lane = threadIdx.x % 32;
    // turn-around: warp wv moves words 4 wv .. 4 wv + 3 of every position, lane l the positions l, l + 32, ...; where a
    // position sits inside a channel's box does not depend on the unit (up to the NCHW column offset, added below)
    int raw_of[U::PER_LANE];
#pragma unroll
    for (int j = 0; j < U::PER_LANE; ++j) {
        const int p = lane + 32 * j;
        raw_of[j] = CHWN_IN ? p : (p / COLS) * BOXW + (p % COLS);
    }
    const long long plane_words = a.tp * a.cp / VEC;
    uint32_t* __restrict__ vw = reinterpret_cast<uint32_t*>(a.v);
    bool aborted = false;
    for (long long i = 0; i < n_my; ++i) {
        const int s = (int)(i % STAGES);
        const bool ok = mbar_wait_bounded(bars + 8 * s, (uint32_t)((i / STAGES) & 1), abort_flag, status, ITP_WAIT_CODE);
        if (!__syncthreads_and(ok)) { aborted = true; break; }
        int c0, xc, q, z;
        decode(i, c0, xc, q, z);
        const int off = CHWN_IN ? 0 : xc * IT_TX * M - a.pad - box_start(xc);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const int w_l = 4 * wv + cc;
#pragma unroll
            for (int j = 0; j < U::PER_LANE; ++j) {
                const int p = lane + 32 * j;
                if (U::POS % 32 == 0 || p < U::POS) {
                    uint32_t word;
                    if constexpr (VEC == 1) {
                        word = reinterpret_cast<const uint32_t*>(smem_planar + s * U::STAGE_BYTES)[w_l * U::RAW + raw_of[j] + off];
                    } else {
                        const unsigned short* raw = reinterpret_cast<const unsigned short*>(smem_planar + s * U::STAGE_BYTES);
                        word = (uint32_t)raw[(2 * w_l) * U::RAW + raw_of[j] + off] | ((uint32_t)raw[(2 * w_l + 1) * U::RAW + raw_of[j] + off] << 16);
                    }
                    tbuf[p * TP + w_l] = word;
                }
            }
        }
        __syncthreads();   // the rows are complete; the box has been read: its slot can take the unit after the next
        if (threadIdx.x == 0 && i + STAGES < n_my) issue(i + STAGES);
        const int c = c0 + lane * VEC;
        long long t;
        bool tile_ok;
        const uint32_t* src = tbuf + lane;
        if (CHWN_IN) {
            const int n_l = xc * IT_NB + wv;
            tile_ok = n_l < a.ns;
            t = ((long long)n_l * a.bny + z) * a.bnx + q;
            src += wv * TP;
        } else {
            const int bx = xc * IT_TX + wv;
            tile_ok = bx < a.bnx;
            t = ((long long)z * a.bny + q) * a.bnx + bx;
            src += wv * M * TP;
        }
        if (tile_ok && c < a.cp)
            transform_words<A, TIn, TOp, false, TP>(src, CHWN_IN ? A * IT_NB : COLS, CHWN_IN ? IT_NB : 1, vw + (t * a.cp + c) / VEC, plane_words);
        __syncthreads();   // the rows are free for the next unit's turn-around
    }
    if (aborted && threadIdx.x == 0) drain_after_abort();
}

// storage whose rows the TMA unit can address: base and every stride a multiple of 16 bytes, and slabs that start on a
// 16-byte boundary of the image axis for CHWN
template <typename TIn>
static bool planar_tma_ok(const wino_conv_desc& d, const ITArgs& a) {
    constexpr int EPV = 16 / (int)sizeof(TIn);
    if (((uintptr_t)a.x & 15) != 0) return false;
    if (d.layout_in == WINO_NCHW) return d.w % EPV == 0;
    if (d.layout_in == WINO_CHWN) return d.n % EPV == 0 && a.n0 % EPV == 0;
    return false;
}

template <int A, bool CHWN_IN, typename TIn, typename TOp>
static int run_planar_tma(const wino_conv_desc& d, const Geometry& g, const ITArgs& a, cudaStream_t st) {
    using U = PlanarUnit<A, CHWN_IN, TIn>;
    static_assert(U::STAGE_BYTES % 128 == 0, "ring slots stay 128-byte aligned");
    const CUtensorMapDataType dt = sizeof(TIn) == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const unsigned long long es = sizeof(TIn);
    CUtensorMap tm;
    int rc;
    if (CHWN_IN) {
        const unsigned long long dims[4] = {(unsigned long long)d.n, (unsigned long long)d.w, (unsigned long long)d.h, (unsigned long long)d.c};
        const unsigned long long strides[3] = {d.n * es, (unsigned long long)d.w * d.n * es, (unsigned long long)d.h * d.w * d.n * es};
        const unsigned box[4] = {(unsigned)IT_NB, (unsigned)A, (unsigned)A, (unsigned)U::CH};
        rc = encode_tensor_map(&tm, dt, 4, a.x, dims, strides, box, false);
    } else {
        const unsigned long long dims[4] = {(unsigned long long)d.w, (unsigned long long)d.h, (unsigned long long)d.c, (unsigned long long)d.n};
        const unsigned long long strides[3] = {d.w * es, (unsigned long long)d.h * d.w * es, (unsigned long long)d.c * d.h * d.w * es};
        const unsigned box[4] = {(unsigned)U::BOXW, (unsigned)A, (unsigned)U::CH, 1u};
        rc = encode_tensor_map(&tm, dt, 4, a.x, dims, strides, box, false);
    }
    if (rc) return rc;
    int* status = nullptr;
    if ((rc = status_word(&status))) return rc;
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(input_transform_planar_tma<A, CHWN_IN, TIn, TOp>, cudaFuncAttributeMaxDynamicSharedMemorySize, U::SMEM);
    });
    WINO_CUDA_CHECK(attr_err);
    const int cchunks = (g.cp + U::CH - 1) / U::CH;
    const int xchunks = CHWN_IN ? (a.ns + IT_NB - 1) / IT_NB : (g.bnx + IT_TX - 1) / IT_TX;
    const long long units = (long long)cchunks * xchunks * g.bny * (CHWN_IN ? g.bnx : a.ns);
    const long long max_ctas = 2LL * sm_count();
    ProfScope prof(STAGE_INPUT, st);
    count_launch();
    input_transform_planar_tma<A, CHWN_IN, TIn, TOp><<<(unsigned)(units < max_ctas ? units : max_ctas), 256, U::SMEM, st>>>(
        tm, a, xchunks, cchunks, units, status);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

// ---- NHWC, aligned pitch: TMA-staged, persistent ------------------------------------------------------------
constexpr int ITT_WAIT_CODE = 5;

// OCC resident CTAs per SM, each with a ring of ITT_STAGES patches: 3 x 2 (default) or 2 x 3 (WINO_ITT_OCC=2)
template <int A, typename TIn, typename TOp, int OCC>
__global__ void __launch_bounds__(256, OCC)
input_transform_nhwc_tma(const __grid_constant__ CUtensorMap tm_x, const ITArgs a, const int bxchunks, const int cchunks,
                         const long long units, int* status) {
    constexpr int M = A - 2;
    constexpr int COLS = M * IT_TX + 2;
    constexpr int VEC = 4 / (int)sizeof(TIn);
    constexpr int CH = 32 * VEC;                       // channels per unit (128 bytes)
    constexpr int STAGE_BYTES = A * COLS * 128;
    constexpr int ITT_STAGES = OCC == 2 ? 3 : 2;
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
            const long long t = ((long long)n_l * a.bny + by) * a.bnx + bx;
            transform_words<A, TIn, TOp>(reinterpret_cast<const uint32_t*>(smem + s * STAGE_BYTES) + (tl * M) * 32 + lane, COLS, 1,
                                         vw + (t * a.cp + c) / VEC, plane_words);
        }
        __syncthreads();   // the slot is free for the load issued at the top of the next iteration
    }
    if (aborted && threadIdx.x == 0) drain_after_abort();
}

// WINO_GENERIC_TRANSFORMS=1 keeps NHWC off the TMA path (testing aid)
static bool force_generic() {
    static const bool v = [] { const char* e = getenv("WINO_GENERIC_TRANSFORMS"); return e && e[0] == '1'; }();
    return v;
}

template <int A, typename TIn, typename TOp, int OCC>
static int run_nhwc_tma(const wino_conv_desc& d, const Geometry& g, const ITArgs& a, cudaStream_t st) {
    constexpr int M = A - 2;
    constexpr int COLS = M * IT_TX + 2;
    constexpr int VEC = 4 / (int)sizeof(TIn);
    constexpr int CH = 32 * VEC;
    constexpr int ITT_STAGES = OCC == 2 ? 3 : 2;
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
        attr_err = cudaFuncSetAttribute(input_transform_nhwc_tma<A, TIn, TOp, OCC>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    });
    WINO_CUDA_CHECK(attr_err);
    const int cchunks = (g.cp + CH - 1) / CH, bxchunks = (g.bnx + IT_TX - 1) / IT_TX;
    const long long units = (long long)a.ns * g.bny * bxchunks * cchunks;
    const long long max_ctas = (long long)OCC * sm_count();
    ProfScope prof(STAGE_INPUT, st);
    count_launch();
    input_transform_nhwc_tma<A, TIn, TOp, OCC><<<(unsigned)(units < max_ctas ? units : max_ctas), 256, SMEM, st>>>(
        tm, a, bxchunks, cchunks, units, status);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

template <int A, typename TIn, typename TOp>
static int run(const wino_conv_desc& d, const Geometry& g, const ITArgs& a, cudaStream_t st) {
    constexpr int CH = 32 * (4 / (int)sizeof(TIn));
    if (d.layout_in == WINO_NHWC && (d.c * sizeof(TIn)) % 16 == 0 && ((uintptr_t)a.x & 15) == 0 && !force_generic()) {
        // measured on B200 (512 -> 512 at 28 x 28, batch 256, BF16): three CTAs with two stages each 0.137 ms, two CTAs with
        // three stages 0.147 ms: the kernel is bound by instruction latency, more resident warps help more than a deeper ring
        static const int occ = [] { const char* e = getenv("WINO_ITT_OCC"); return e ? atoi(e) : 3; }();
        return occ == 2 ? run_nhwc_tma<A, TIn, TOp, 2>(d, g, a, st) : run_nhwc_tma<A, TIn, TOp, 3>(d, g, a, st);
    }
    // NCHW / CHWN whose rows the TMA unit can address: channel planes staged by TMA (WINO_GENERIC_TRANSFORMS=1 keeps the kernels below)
    if (!force_generic() && planar_tma_ok<TIn>(d, a))
        return d.layout_in == WINO_CHWN ? run_planar_tma<A, true, TIn, TOp>(d, g, a, st) : run_planar_tma<A, false, TIn, TOp>(d, g, a, st);
    const int cchunks = (g.cp + CH - 1) / CH;
    ProfScope prof(STAGE_INPUT, st);
    count_launch();
    if (d.layout_in == WINO_CHWN) {
        dim3 grid((unsigned)(((a.ns + IT_NB - 1) / IT_NB) * cchunks), (unsigned)g.bnx, (unsigned)g.bny);
        input_transform_batch<A, TIn, TOp><<<grid, 256, 0, st>>>(a, cchunks);
    } else {
        const int bxchunks = (g.bnx + IT_TX - 1) / IT_TX;
        dim3 grid((unsigned)(bxchunks * cchunks), (unsigned)g.bny, (unsigned)a.ns);
        if (d.layout_in == WINO_NCHW)
            input_transform_strip<A, true, TIn, TOp><<<grid, 256, 0, st>>>(a, bxchunks, cchunks);
        else
            input_transform_strip<A, false, TIn, TOp><<<grid, 256, 0, st>>>(a, bxchunks, cchunks);
    }
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

template <int A>
static int dispatch(const wino_conv_desc& d, const Geometry& g, const ITArgs& a, cudaStream_t st) {
    switch (g.operand) {
        case OP_F32: return run<A, float, float>(d, g, a, st);
        case OP_TF32: return run<A, float, tf32_t>(d, g, a, st);
        case OP_TF32X3: return run<A, float, float>(d, g, a, st);   // plain FP32 V: the tile GEMM splits it
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

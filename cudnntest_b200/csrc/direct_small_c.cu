// Direct 3x3 convolution for very thin inputs (C <= 3: the first VGG layer, 3 -> 64 at 224 x 224), sm_100a.
//
// The reference sends this layer through the same Winograd pipeline with the channel count padded to 8
// (comparison/layoutCompare.cu:43-46 "layer 1: c = 3", KSize rounding wrapedConv_NCHW.cuh:362).  With three
// channels the 36 products per tile cost far more memory traffic than the convolution itself, so this library
// routes the tensor-core variants of such layers to an implicit-GEMM kernel instead: the contraction is the
// 9*C <= 27 taps, padded to 32.
//
//   * one thread = one output pixel.  It gathers its 3x3xC patch (zero padded) straight from the input layout
//     and writes it as one K-major row of a 128 x 32 operand tile in shared memory, in the 128-byte-swizzled
//     layout tcgen05.mma reads;
//   * the 64 x 32 filter tile is built once per CTA the same way;
//   * thread 0 issues tcgen05.mma (M = 128 pixels, N = 64 filters, K = 32) into a 64-column accumulator in tensor
//     memory and commits to an mbarrier.  The bias is the 28th contraction slot (pixel rows hold 1, filter rows the
//     bias rounded to the operand format), so the MMA adds it;
//   * every thread then reads its own accumulator lane (tcgen05.ld) and applies ReLU; for dense NHWC output each
//     warp turns its 32 pixels x 64 outputs around in shared memory so that a store instruction writes four whole
//     128-byte lines, other layouts store element by element.
// Several CTAs share an SM so one CTA's gather overlaps another's MMA and stores.  Bound: HBM, by the output
// write (N*K*OH*OW elements); the input is read once from HBM and nine times from L1/L2.
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace wino {

namespace {

constexpr int DC_WAIT_CODE = 21;

struct DCArgs {
    const void* x;
    const void* w;
    const float* bias;
    void* y;
    int N, C, H, W, K, pad;
    int oh, ow;
    long long pixels;      // N * oh * ow
    int relu;
    int n_fastest;         // pixel order of a tile: images fastest (CHWN) or columns fastest
    int tma_store;         // dense NHWC 2-byte output: tiles leave through TMA stores of the staging rows
    uint32_t idesc;
    Strides sx, sw, sy;
    int* status;
};

template <typename TIn>
struct OperandRow;
// BF16 storage: operands are the stored bf16 values themselves, moved as raw 16-bit patterns
// (32 x 2 bytes = four 16-byte chunks per row)
template <>
struct OperandRow<__nv_bfloat16> {
    static constexpr bool TF32 = false;
    using raw_t = unsigned short;
    static __device__ __forceinline__ raw_t load(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const unsigned short*>(p)); }
    static __device__ __forceinline__ raw_t zero() { return 0; }
    static __device__ __forceinline__ raw_t one() { return 0x3F80; }
    static __device__ __forceinline__ raw_t from_f32(float f) { return __bfloat16_as_ushort(__float2bfloat16_rn(f)); }
    static __device__ __forceinline__ void store(uint8_t* row_base, int row, const raw_t (&v)[32]) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint32_t wds[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) wds[e] = (uint32_t)v[8 * c + 2 * e] | ((uint32_t)v[8 * c + 2 * e + 1] << 16);
            *reinterpret_cast<uint4*>(row_base + ((c ^ (row & 7)) << 4)) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
        }
    }
};
// float storage: operands rounded to TF32 (32 x 4 bytes = eight chunks per row)
template <>
struct OperandRow<float> {
    static constexpr bool TF32 = true;
    using raw_t = float;
    static __device__ __forceinline__ raw_t load(const float* p) { return from_float<tf32_t>(__ldg(p)).v; }
    static __device__ __forceinline__ raw_t zero() { return 0.f; }
    static __device__ __forceinline__ raw_t one() { return 1.f; }
    static __device__ __forceinline__ raw_t from_f32(float f) { return from_float<tf32_t>(f).v; }
    static __device__ __forceinline__ void store(uint8_t* row_base, int row, const raw_t (&v)[32]) {
#pragma unroll
        for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(row_base + ((c ^ (row & 7)) << 4)) =
                make_uint4(__float_as_uint(v[4 * c]), __float_as_uint(v[4 * c + 1]), __float_as_uint(v[4 * c + 2]), __float_as_uint(v[4 * c + 3]));
    }
};

template <typename TIn, typename TOut, int CC>
__global__ void __launch_bounds__(128, 5) direct_small_c_kernel(const __grid_constant__ CUtensorMap tm_y, const DCArgs a) {
    using Row = OperandRow<TIn>;
    using raw_t = typename Row::raw_t;
    constexpr int BIAS_COL = 9 * CC;        // first unused contraction slot: pixel rows hold 1 there, filter rows the bias
    static_assert(BIAS_COL < 32, "the contraction is padded to 32 and one spare slot carries the bias");
    // two operand tiles used alternately: while the MMA / the output store of one tile still reads its buffer, the
    // next tile is gathered into the other
    __shared__ __align__(1024) uint8_t a_tiles[2][128 * 128];
    __shared__ __align__(1024) uint8_t b_tile[64 * 128];
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;

    const int tid = threadIdx.x, warp = tid / 32;
    const int k0 = blockIdx.y * 64;
    const uint32_t bar = smem_u32(&bar_storage);

    if (tid == 0) {
        mbar_init(bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), 64);
    // dense NHWC output with a whole, 16-byte aligned block of 64 filters: pixels are consecutive 2*K-byte (4*K) rows
    const bool dense_nhwc = !a.n_fastest && a.sy.c == 1 && a.sy.w == a.K && a.sy.h == (long long)a.ow * a.K &&
                            a.sy.n == (long long)a.oh * a.ow * a.K && k0 + 64 <= a.K &&
                            ((reinterpret_cast<uintptr_t>(a.y) | (uintptr_t)(a.K * sizeof(TOut)) | (uintptr_t)(k0 * sizeof(TOut))) & 15) == 0;

    // barrier set-up and the tensor-memory allocation overlapped the previous kernel's last wave; every tensor (the
    // packed filters too: the kernel that packs them may be the one just before this one) is touched from here on
    pdl_launch_dependents();
    pdl_wait();
    // filter tile: row kf = packed filter row k0 + kf (32 operand values, see pack_direct_filters), zero beyond K;
    // the bias rides in the spare contraction slot (rounded to the operand format: it is added by the MMA itself)
    if (tid < 64) {
        raw_t v[32];
        const int kf = k0 + tid;
        const TIn* wp = reinterpret_cast<const TIn*>(a.w) + (long long)kf * 32;
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = kf < a.K ? Row::load(wp + i) : Row::zero();
        v[BIAS_COL] = (a.bias && kf < a.K) ? Row::from_f32(__ldg(a.bias + kf)) : Row::zero();
        Row::store(b_tile + tid * 128, tid, v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    const uint32_t a_s0 = smem_u32(a_tiles[0]), b_s = smem_u32(b_tile);
    const TIn* __restrict__ xin = reinterpret_cast<const TIn*>(a.x);
    TOut* __restrict__ yout = reinterpret_cast<TOut*>(a.y);

    uint32_t parity = 0;
    const long long tiles = (a.pixels + 127) / 128;
    const bool idx32 = a.pixels < (1LL << 31);
    // dense NHWC input with exactly three channels, 4-byte aligned
    const bool nhwc3_in = !a.n_fastest && a.C == 3 && a.sx.c == 1 && a.sx.w == 3 && a.sx.h == 3LL * a.W && a.sx.n == 3LL * a.W * a.H &&
                          (reinterpret_cast<uintptr_t>(a.x) & 3) == 0 && a.W >= 4 && a.pad <= 1;
    const bool use_tma = sizeof(TOut) == 2 && a.tma_store && dense_nhwc;
    int buf = 0;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x, buf ^= 1) {
        uint8_t* a_tile = a_tiles[buf];
        const uint32_t a_s = a_s0 + (uint32_t)buf * (128 * 128);
        if (use_tma) {          // the store that last read this buffer (two tiles ago) must be done with it
            if ((tid & 31) == 0) tma_store_wait_read<1>();
            __syncwarp();
        }
        const long long p = tile * 128 + tid;
        const bool valid = p < a.pixels;
        int n = 0, oy = 0, ox = 0;
        if (valid) {
            // pixel index -> (image, row, column): 32-bit arithmetic whenever the tensor allows it
            const int inner = a.n_fastest ? a.N : a.ow, mid = a.n_fastest ? a.ow : a.oh;
            int i0, i1, i2;
            if (idx32) {
                const unsigned q = (unsigned)p, q1 = q / (unsigned)inner;
                i0 = (int)(q - q1 * (unsigned)inner);
                i2 = (int)(q1 / (unsigned)mid);
                i1 = (int)(q1 - (unsigned)i2 * (unsigned)mid);
            } else {
                i0 = (int)(p % inner);
                const long long q1 = p / inner;
                i1 = (int)(q1 % mid);
                i2 = (int)(q1 / mid);
            }
            if (a.n_fastest) { n = i0; ox = i1; oy = i2; }     // CHWN: consecutive threads take consecutive images of one output position
            else { ox = i0; oy = i1; n = i2; }
        }
        bool fast = false;
        if constexpr (sizeof(TIn) == 2 && CC == 3) {
            // Dense NHWC input with exactly three channels: the nine taps of a filter row are 18 contiguous bytes.
            // A pixel fetches them as five aligned 32-bit words per row and shifts them into place (the start is only
            // 2-byte aligned).  On the left / right image border the words still come from inside the tensor (the
            // neighbouring row's end or start) and the taps that fall into the padding are masked to zero; only the
            // pixels whose words would leave the tensor (its very first and last ones) take the element-wise gather.
            const bool left_ok = ox - a.pad >= 0, right_ok = ox + 2 - a.pad < a.W;
            fast = valid && nhwc3_in && !(n == 0 && oy - a.pad <= 0 && !left_ok) &&
                   !(n == a.N - 1 && oy + 2 - a.pad >= a.H - 1 && ox + 3 - a.pad >= a.W);
            if (fast) {
                const long long m_pix = ((long long)n * a.H * a.W + (ox - a.pad)) * 3;       // element offset of tap (row 0 of the image, s = 0)
                uint32_t st[3][5];
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    const int ih = oy + r - a.pad;
                    const bool row_ok = ih >= 0 && ih < a.H;
                    const long long m0 = m_pix + (long long)(row_ok ? ih : 0) * a.W * 3;
                    const uint32_t* wp = reinterpret_cast<const uint32_t*>(xin) + (m0 >> 1);
                    const uint32_t sh = (uint32_t)(m0 & 1) * 16;
                    uint32_t aw[5];
#pragma unroll
                    for (int k = 0; k < 5; ++k) aw[k] = row_ok ? __ldg(wp + k) : 0u;
#pragma unroll
                    for (int k = 0; k < 4; ++k) st[r][k] = __funnelshift_r(aw[k], aw[k + 1], sh);
                    st[r][4] = aw[4] >> sh;
                    if (!left_ok) { st[r][0] = 0u; st[r][1] &= 0xFFFF0000u; }      // taps 0..2 (s = 0) are padding
                    if (!right_ok) { st[r][3] = 0u; st[r][4] = 0u; }               // taps 6..8 (s = 2) are padding
                }
                // operand row: elements 0..8 = filter row 0, 9..17 = row 1, 18..26 = row 2, 27 = 1 (bias slot), 28..31 = 0
                uint32_t w[16];
#pragma unroll
                for (int k = 0; k < 4; ++k) w[k] = st[0][k];
                w[4] = (st[0][4] & 0xFFFFu) | (st[1][0] << 16);
#pragma unroll
                for (int k = 0; k < 4; ++k) w[5 + k] = __funnelshift_r(st[1][k], st[1][k + 1], 16);
#pragma unroll
                for (int k = 0; k < 4; ++k) w[9 + k] = st[2][k];
                w[13] = (st[2][4] & 0xFFFFu) | ((uint32_t)Row::one() << 16);
                w[14] = 0u; w[15] = 0u;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(a_tile + tid * 128 + ((c ^ (tid & 7)) << 4)) = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
            }
        }
        if (!fast) {
            raw_t v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = Row::zero();
            if (valid) {
                const TIn* xp = xin + n * a.sx.n;
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    const int ih = oy + r - a.pad;
                    if (ih < 0 || ih >= a.H) continue;
#pragma unroll
                    for (int s = 0; s < 3; ++s) {
                        const int iw = ox + s - a.pad;
                        if (iw < 0 || iw >= a.W) continue;
#pragma unroll
                        for (int c = 0; c < CC; ++c)
                            if (c < a.C) v[(r * 3 + s) * CC + c] = Row::load(xp + c * a.sx.c + ih * a.sx.h + iw * a.sx.w);
                    }
                }
                v[BIAS_COL] = Row::one();
            }
            Row::store(a_tile + tid * 128, tid, v);
        }
        fence_async_shared();        // the tile was written through the generic proxy, tcgen05.mma reads it through the async proxy
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 4 / (Row::TF32 ? 1 : 2); ++ks)
                tc_mma<Row::TF32>(tmem_base, smem_desc_k128(a_s + ks * 32), smem_desc_k128(b_s + ks * 32), a.idesc, ks ? 1u : 0u);
            tc_commit(bar);
        }
        bool ok = mbar_wait_bounded(bar, parity, &abort_flag, a.status, DC_WAIT_CODE);
        parity ^= 1;
        if (!__syncthreads_and(ok)) break;
        tc_fence_after();
        uint32_t r0[32], r1[32];
        const uint32_t lane_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
        tmem_ld_32x32(lane_addr, r0);
        tmem_ld_32x32(lane_addr + 32, r1);
        tmem_ld_wait();
        tc_fence_before();
        __syncthreads();             // accumulator and operand tile may be overwritten by the next tile from here on
        if (dense_nhwc) {
            // Each lane holds one pixel's 64 outputs.  Stored straight from there, one 16-byte store instruction of a warp
            // touches 32 different 128-byte lines; instead the warp turns its 32 x 128-byte block around in its own rows
            // of the operand tile (free once the MMA has completed, chunk index XOR row to stay conflict-free) so that
            // eight consecutive lanes write one pixel's 128 contiguous bytes: four full lines per instruction.
            constexpr int PER = 16 / (int)sizeof(TOut);          // outputs per 16-byte chunk
            constexpr int PASSES = 64 / (8 * PER);               // 128 bytes of a pixel per pass
            uint8_t* wtile = a_tile + warp * 32 * 128;
            const int lane = tid & 31;
            const long long p0 = tile * 128 + warp * 32;
            TOut* ybase = yout + p0 * a.K + k0;
            const int rows_left = (int)(a.pixels - p0 < 32 ? a.pixels - p0 : 32);
#pragma unroll
            for (int pass = 0; pass < PASSES; ++pass) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    uint32_t wds[4];
                    if constexpr (sizeof(TOut) == 2) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int kk = c * 8 + 2 * e;         // one pass: 64 filters
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(kk < 32 ? r0[kk] : r1[kk - 32]),
                                                                     __uint_as_float(kk + 1 < 32 ? r0[kk + 1] : r1[kk + 1 - 32]));
                            if (a.relu) h = __hmax2(h, __floats2bfloat162_rn(0.f, 0.f));   // ReLU commutes with the rounding
                            wds[e] = *reinterpret_cast<uint32_t*>(&h);
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int kk = pass * 32 + c * 4 + e;
                            const float val = __uint_as_float(kk < 32 ? r0[kk] : r1[kk - 32]);
                            wds[e] = __float_as_uint(a.relu ? fmaxf(val, 0.f) : val);
                        }
                    }
                    *reinterpret_cast<uint4*>(wtile + lane * 128 + ((c ^ (lane & 7)) << 4)) = make_uint4(wds[0], wds[1], wds[2], wds[3]);
                }
                if (use_tma) {      // the staging rows are already a 128-byte-swizzled box: one lane hands them to the TMA unit
                    fence_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_y, smem_u32(wtile), k0, (int)p0);
                        tma_store_commit();
                    }
                    continue;
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int j = i * 4 + (lane >> 3), cc = lane & 7;
                    const uint4 v4 = *reinterpret_cast<const uint4*>(wtile + j * 128 + ((cc ^ (j & 7)) << 4));
                    if (j < rows_left)
                        *reinterpret_cast<uint4*>(ybase + j * a.K + pass * 8 * PER + cc * PER) = v4;
                }
                __syncwarp();
            }
        } else if (valid) {
            // any other output layout, or a ragged block of filters: one element at a time
            TOut* yp = yout + n * a.sy.n + oy * a.sy.h + ox * a.sy.w;
#pragma unroll
            for (int kk = 0; kk < 64; ++kk) {
                if (k0 + kk >= a.K) break;
                float val = __uint_as_float(kk < 32 ? r0[kk] : r1[kk - 32]);
                if (a.relu) val = fmaxf(val, 0.f);
                yp[(long long)(k0 + kk) * a.sy.c] = from_float<TOut>(val);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 64);
    }
}

// Packed filters for the kernel above: P[k][(r*3 + s)*3 + c] = w[k][c][r][s] through the filter layout's strides,
// 32 values per filter (zero beyond the 9*C taps), in the operand format (bf16, or float rounded to TF32).
template <typename TIn, bool EXACT = false>
__global__ void pack_direct_filters(const TIn* __restrict__ w, TIn* __restrict__ out, int K, int C, Strides sw) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= K * 32) return;
    const int k = idx / 32, col = idx % 32;
    const int rs = col / 3, c = col % 3;
    float v = 0.f;
    if (rs < 9 && c < C) v = to_float<TIn>(w[k * sw.n + c * sw.c + (rs / 3) * sw.h + (rs % 3) * sw.w]);
    if (sizeof(TIn) == 4 && !EXACT) v = from_float<tf32_t>(v).v;
    out[idx] = from_float<TIn>(v);
}

// Exact-FP32 variant (FFMA, no tensor cores) of the same idea for the float path: one thread = one output pixel and a
// block of 64 filters.  The 27 taps sit in registers, the filter block in shared memory as [tap][filter] so that a
// 16-byte broadcast read feeds four filters; each product is one FP32 fused multiply-add, taps accumulated in
// (r, s, c) order on top of the bias.  The Winograd pipeline pads these three channels to eight and moves 36 + 36
// transform-domain planes through HBM for them (1.40 ms at batch 64 against 0.68 ms for cuDNN).
template <int CC>
__global__ void __launch_bounds__(128) direct_small_c_fp32_kernel(const DCArgs a) {
    constexpr int TAPS = 9 * CC;
    __shared__ __align__(16) float ws[TAPS][64];
    __shared__ __align__(16) float bias_s[64];
    const int tid = threadIdx.x;
    const int k0 = blockIdx.y * 64;
    const float* __restrict__ wpk = reinterpret_cast<const float*>(a.w);      // packed [K][32]
    for (int i = tid; i < TAPS * 64; i += 128) {
        const int t = i / 64, k = i % 64;
        ws[t][k] = k0 + k < a.K ? __ldg(wpk + (long long)(k0 + k) * 32 + t) : 0.f;
    }
    if (tid < 64) bias_s[tid] = (a.bias && k0 + tid < a.K) ? __ldg(a.bias + k0 + tid) : 0.f;
    __syncthreads();
    const float* __restrict__ xin = reinterpret_cast<const float*>(a.x);
    float* __restrict__ yout = reinterpret_cast<float*>(a.y);
    const bool dense_nhwc = a.sy.c == 1 && k0 + 64 <= a.K && ((reinterpret_cast<uintptr_t>(a.y) | (uintptr_t)(a.K * 4) | (uintptr_t)(k0 * 4)) & 15) == 0 &&
                            a.sy.w % 4 == 0 && a.sy.h % 4 == 0 && a.sy.n % 4 == 0;
    const long long tiles = (a.pixels + 127) / 128;
    for (long long tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
        const long long p = tile * 128 + tid;
        if (p >= a.pixels) continue;
        int n, oy, ox;
        {
            const int inner = a.n_fastest ? a.N : a.ow, mid = a.n_fastest ? a.ow : a.oh;
            const int i0 = (int)(p % inner);
            const long long q1 = p / inner;
            const int i1 = (int)(q1 % mid), i2 = (int)(q1 / mid);
            if (a.n_fastest) { n = i0; ox = i1; oy = i2; }
            else { ox = i0; oy = i1; n = i2; }
        }
        float v[TAPS];
#pragma unroll
        for (int i = 0; i < TAPS; ++i) v[i] = 0.f;
        const float* xp = xin + n * a.sx.n;
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            const int ih = oy + r - a.pad;
            if (ih < 0 || ih >= a.H) continue;
#pragma unroll
            for (int s = 0; s < 3; ++s) {
                const int iw = ox + s - a.pad;
                if (iw < 0 || iw >= a.W) continue;
#pragma unroll
                for (int c = 0; c < CC; ++c)
                    if (c < a.C) v[(r * 3 + s) * CC + c] = __ldg(xp + c * a.sx.c + ih * a.sx.h + iw * a.sx.w);
            }
        }
        float* yp = yout + n * a.sy.n + oy * a.sy.h + ox * a.sy.w;
#pragma unroll 1
        for (int kb = 0; kb < 64; kb += 16) {       // 16 filters at a time keep the accumulators in registers
            float2 acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = make_float2(bias_s[kb + 2 * j], bias_s[kb + 2 * j + 1]);
#pragma unroll
            for (int t = 0; t < TAPS; ++t) {
                const float2 at = make_float2(v[t], v[t]);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 w4 = *reinterpret_cast<const float4*>(&ws[t][kb + 4 * q]);
                    acc[2 * q] = __ffma2_rn(at, make_float2(w4.x, w4.y), acc[2 * q]);
                    acc[2 * q + 1] = __ffma2_rn(at, make_float2(w4.z, w4.w), acc[2 * q + 1]);
                }
            }
            if (a.relu) {
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[j] = make_float2(fmaxf(acc[j].x, 0.f), fmaxf(acc[j].y, 0.f));
            }
            if (dense_nhwc) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    *reinterpret_cast<float4*>(yp + k0 + kb + 4 * q) = make_float4(acc[2 * q].x, acc[2 * q].y, acc[2 * q + 1].x, acc[2 * q + 1].y);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (k0 + kb + j < a.K) yp[(long long)(k0 + kb + j) * a.sy.c] = (j & 1) ? acc[j / 2].y : acc[j / 2].x;
            }
        }
    }
}

template <typename TIn, typename TOut>
int run(DCArgs a, cudaStream_t st) {
    const long long tiles = (a.pixels + 127) / 128;
    const long long max_ctas = 5LL * sm_count();
    dim3 grid((unsigned)(tiles < max_ctas ? tiles : max_ctas), (unsigned)((a.K + 63) / 64));
    // dense NHWC 2-byte output seen as a [pixels][K] matrix: 32-pixel x 64-filter boxes, 128-byte swizzle
    CUtensorMap tm_y;
    memset(&tm_y, 0, sizeof(tm_y));
    a.tma_store = 0;
    static const bool tma_off = [] { const char* e = getenv("WINO_THIN_TMA_STORE"); return e && e[0] == '0'; }();
    if (!tma_off && sizeof(TOut) == 2 && !a.n_fastest && a.sy.c == 1 && a.sy.w == a.K && a.sy.h == (long long)a.ow * a.K &&
        a.sy.n == (long long)a.oh * a.ow * a.K && a.K % 8 == 0 && a.pixels < (1LL << 31) && ((uintptr_t)a.y & 15) == 0) {
        const unsigned long long dims[2] = {(unsigned long long)a.K, (unsigned long long)a.pixels};
        const unsigned long long strides[1] = {(unsigned long long)a.K * 2ull};
        const unsigned box[2] = {64u, 32u};
        if (encode_tensor_map(&tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a.y, dims, strides, box, true) == WINO_OK) a.tma_store = 1;
    }
    ProfScope prof(STAGE_DIRECT, st);
    count_launch();
    WINO_CUDA_CHECK(launch_kernel(direct_small_c_kernel<TIn, TOut, 3>, grid, dim3(128), 0, st, pdl_enabled(), tm_y, a));
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace

bool direct_small_c_applies(const wino_conv_desc& d) {
    static const bool off = [] { const char* e = getenv("WINO_NO_DIRECT"); return e && e[0] == '1'; }();
    return !off && d.wino == 0 && d.c <= 3 && !d.pool2x2 && !out_type_differs(d);
}

size_t direct_small_c_filter_bytes(const wino_conv_desc& d) { return (size_t)d.k * 32 * (d.dtype == WINO_BF16 ? 2 : 4); }

int launch_direct_small_c_pack(const wino_conv_desc& d, const void* w, void* packed, cudaStream_t st) {
    const int total = d.k * 32;
    const Strides sw = filter_strides(d.layout_in, d.k, d.c);
    ProfScope prof(STAGE_FILTER, st);
    count_launch();
    if (d.dtype == WINO_BF16)
        pack_direct_filters<__nv_bfloat16><<<(total + 255) / 256, 256, 0, st>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)packed, d.k, d.c, sw);
    else if (d.dtype == WINO_TF32)   // WINO_FP32 and WINO_FP32X3 both take the exact kernel below
        pack_direct_filters<float><<<(total + 255) / 256, 256, 0, st>>>((const float*)w, (float*)packed, d.k, d.c, sw);
    else        // exact FP32: the filters stay unrounded
        pack_direct_filters<float, true><<<(total + 255) / 256, 256, 0, st>>>((const float*)w, (float*)packed, d.k, d.c, sw);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

// `w` is the packed filter buffer written by launch_direct_small_c_pack
int launch_direct_small_c(const wino_conv_desc& d, const Geometry& g, const void* x, const void* w, const float* bias,
                          void* y, cudaStream_t st) {
    DCArgs a;
    a.x = x; a.w = w; a.bias = d.has_bias ? bias : nullptr; a.y = y;
    a.N = d.n; a.C = d.c; a.H = d.h; a.W = d.w; a.K = d.k; a.pad = d.pad;
    a.oh = g.oh; a.ow = g.ow;
    a.pixels = (long long)d.n * g.oh * g.ow;
    a.relu = d.relu;
    a.n_fastest = d.layout_in == WINO_CHWN || d.layout_out == WINO_CHWN;
    a.idesc = make_idesc(d.dtype == WINO_TF32 ? OP_TF32 : OP_BF16, 64);
    a.sx = act_strides(d.layout_in, d.n, d.c, d.h, d.w);
    a.sw = filter_strides(d.layout_in, d.k, d.c);   // unused by the kernel: the filters arrive packed
    a.sy = act_strides(d.layout_out, d.n, d.k, g.oh, g.ow);
    if (a.pixels == 0) return WINO_OK;
    if (d.dtype == WINO_FP32 || d.dtype == WINO_FP32X3) {
        const long long tiles = (a.pixels + 127) / 128;
        const long long max_ctas = 8LL * sm_count();
        dim3 grid((unsigned)(tiles < max_ctas ? tiles : max_ctas), (unsigned)((a.K + 63) / 64));
        a.status = nullptr;
        ProfScope prof(STAGE_DIRECT, st);
        count_launch();
        direct_small_c_fp32_kernel<3><<<grid, 128, 0, st>>>(a);
        WINO_CUDA_CHECK(cudaGetLastError());
        return WINO_OK;
    }
    int rc = status_word(&a.status);
    if (rc) return rc;
    return d.dtype == WINO_BF16 ? run<__nv_bfloat16, __nv_bfloat16>(a, st) : run<float, float>(a, st);
}

}  // namespace wino

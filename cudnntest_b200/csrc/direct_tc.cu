// Direct (implicit-GEMM) 3x3 convolution on tcgen05 for thin, large-spatial NHWC BF16 layers (C = 64, 128), sm_100a.
//
// Why it exists: for C <= 128 the Winograd pipeline is bound by writing and re-reading its transform-domain
// buffers (V and the products are 2.25x / 1.5x the size of the activations), while the direct convolution of such
// a layer only has to read x and write y once and its 9x larger tensor work is still far below the tensor roof.
// The reference has a direct convolution of the same shape of idea on CUDA cores that it never launches
// (Conv_fuse, fusedTest/winotrans.cuh:1868-1992); its live path sends every layer through Winograd.
//
//   * output tile = 8 (w) x 16 (h) pixels of one image = the 128 rows of the MMA; filters in blocks of BN;
//   * per 64-channel chunk ONE 4-D cp.async.bulk.tensor load brings the 16 (w) x 18 (h) x 128-byte halo box of the
//     tile into a 128-byte-swizzled ring slot (zero padding = the TMA unit's out-of-range fill).  The operand of
//     filter tap (r, s) is that same slot read through a shared-memory matrix descriptor that starts at pixel
//     (r, s) of the box: 8-pixel row groups 2048 bytes apart, start address advanced by (16 r + s) * 128 bytes
//     (the swizzle phase follows the address).  Nine taps x four K-steps of tcgen05.mma per chunk reuse one load;
//   * filter tiles Wd[tap][K][Cp] are either resident in shared memory for the whole kernel (C = 64: nine tiles) or
//     streamed through their own ring;
//   * epilogue warps read their accumulator lane (= pixel) from tensor memory, add bias, apply ReLU and, for
//     block-ending layers, take the 2x2 max with two warp shuffles (the tile's pixel order puts the 2x2 window in
//     lanes l, l^1, l^8, l^9), then store 16-byte vectors of the pixel's BN contiguous NHWC channels.
// Bound: tensor pipe (2*N*K*C*OH*OW*9 flops) once the loads are hidden; HBM traffic is x + y only.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"
#include "direct_tc.cuh"

namespace wino {

namespace {

template <int BN, int A_STAGES, int B_STAGES, bool B_RESIDENT>
struct DtSmem {
    static constexpr int B_TILE = BN * 128;
    static constexpr int A_OFF = 0;
    static constexpr int B_OFF = A_OFF + A_STAGES * DT_A_STRIDE;
    static constexpr int B_BYTES = (B_RESIDENT ? 9 : B_STAGES) * B_TILE;       // resident: the 9 taps of a single-chunk layer
    static constexpr int BAR_OFF = B_OFF + B_BYTES;
    static constexpr int NBARS = 2 * A_STAGES + 2 * B_STAGES + 4 + 1;
    static constexpr int SLOT_OFF = BAR_OFF + 8 * NBARS;
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;
};

template <int BN, int A_STAGES, int B_STAGES, bool B_RESIDENT>
__global__ void __launch_bounds__(DT_THREADS, 1)
direct_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const DtParams p) {
    using L = DtSmem<BN, A_STAGES, B_STAGES, B_RESIDENT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFF;
    const uint32_t bar_afull = bars, bar_aempty = bar_afull + 8 * A_STAGES;
    const uint32_t bar_bfull = bar_aempty + 8 * A_STAGES, bar_bempty = bar_bfull + 8 * B_STAGES;
    const uint32_t bar_tfull = bar_bempty + 8 * B_STAGES, bar_tempty = bar_tfull + 16, bar_bres = bar_tempty + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::SLOT_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::SLOT_OFF + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; ++s) { mbar_init(bar_afull + 8 * s, 1); mbar_init(bar_aempty + 8 * s, 1); }
        for (int s = 0; s < B_STAGES; ++s) { mbar_init(bar_bfull + 8 * s, 1); mbar_init(bar_bempty + 8 * s, 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 32 * DT_EPI_WARPS); }
        mbar_init(bar_bres, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), 2 * BN < 32 ? 32 : 2 * BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long tiles_img = (long long)p.tiles_x * p.tiles_y;
    const long long total = (long long)p.N * tiles_img * p.nblocks;
    // with resident filters a CTA keeps one filter block: it only walks tiles of its own nb
    const int my_nb = B_RESIDENT ? (int)(blockIdx.x % p.nblocks) : 0;

    auto decode = [&](long long t, int& n, int& ty, int& tx, int& nb) {
        nb = (int)(t % p.nblocks); t /= p.nblocks;
        tx = (int)(t % p.tiles_x); t /= p.tiles_x;
        ty = (int)(t % p.tiles_y);
        n = (int)(t / p.tiles_y);
    };
    const long long first = B_RESIDENT ? (long long)(blockIdx.x / p.nblocks) * p.nblocks + my_nb : blockIdx.x;
    const long long step = B_RESIDENT ? (long long)(gridDim.x / p.nblocks) * p.nblocks : gridDim.x;

    if (warp == 0) {
        {   // the whole warp walks the rings (warp-uniform addresses); one elected lane issues the copies
            const bool issuer = elect_one();
            bool ok = true;
            if (B_RESIDENT) {       // all taps and chunks of this CTA's filter block, once
                if (issuer) mbar_arrive_expect_tx(bar_bres, (uint32_t)(9 * p.cchunks * L::B_TILE));
                for (int ch = 0; ch < p.cchunks; ++ch)
                    for (int tap = 0; tap < 9; ++tap)
                        if (issuer) tma_load_3d(base + L::B_OFF + (ch * 9 + tap) * L::B_TILE, &tm_w, bar_bres, ch * 64, my_nb * BN, tap);
            }
            unsigned long long acount = 0, bcount = 0;
            for (long long t = first; ok && t < total; t += step) {
                int n, ty, tx, nb;
                decode(t, n, ty, tx, nb);
                for (int ch = 0; ok && ch < p.cchunks; ++ch) {
                    const int st = (int)(acount % A_STAGES);
                    if (!mbar_wait_warp(bar_aempty + 8 * st, (uint32_t)(((acount / A_STAGES) & 1) ^ 1), abort_flag, p.status, DT_W_A_EMPTY)) { ok = false; break; }
                    if (issuer) mbar_arrive_expect_tx(bar_afull + 8 * st, DT_A_BYTES);
                    if (issuer) tma_load_4d(base + L::A_OFF + st * DT_A_STRIDE, &tm_x, bar_afull + 8 * st, ch * 64, tx * DT_TW - p.pad, ty * DT_TH - p.pad, n);
                    ++acount;
                    if (!B_RESIDENT) {
                        for (int tap = 0; tap < 9; ++tap) {
                            const int sb = (int)(bcount % B_STAGES);
                            if (!mbar_wait_warp(bar_bempty + 8 * sb, (uint32_t)(((bcount / B_STAGES) & 1) ^ 1), abort_flag, p.status, DT_W_B_EMPTY)) { ok = false; break; }
                            if (issuer) mbar_arrive_expect_tx(bar_bfull + 8 * sb, L::B_TILE);
                            if (issuer) tma_load_3d(base + L::B_OFF + sb * L::B_TILE, &tm_w, bar_bfull + 8 * sb, ch * 64, nb * BN, tap);
                            ++bcount;
                        }
                    }
                }
            }
            if (!ok && issuer) drain_after_abort();
        }
    } else if (warp == 1) {
        {   // warp-uniform loop, one elected lane issues: from a single-lane branch every tcgen05.mma cost its thread tens of cycles
            const bool issuer = elect_one();
            bool ok = true;
            if (B_RESIDENT) ok = mbar_wait_warp(bar_bres, 0, abort_flag, p.status, DT_W_B_RESIDENT);
            unsigned long long acount = 0, bcount = 0;
            int as = 0;
            uint32_t aphase = 0;
            for (long long t = first; ok && t < total; t += step) {
                if (!mbar_wait_warp(bar_tempty + 8 * as, aphase ^ 1, abort_flag, p.status, DT_W_T_EMPTY)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
                for (int ch = 0; ok && ch < p.cchunks; ++ch) {
                    const int st = (int)(acount % A_STAGES);
                    if (!mbar_wait_warp(bar_afull + 8 * st, (uint32_t)((acount / A_STAGES) & 1), abort_flag, p.status, DT_W_A_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_s = base + L::A_OFF + st * DT_A_STRIDE;
                    // descriptors are built once per ring slot; per tap and K-step only a constant is added to the
                    // 16-byte-unit start address in the low word (the single issuing lane is the critical path)
                    const uint64_t a_desc0 = smem_desc_k128_sbo(a_s, DT_BOX_W * 128);
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        uint64_t b_desc0;
                        int sb = 0;
                        if (B_RESIDENT) {
                            b_desc0 = smem_desc_k128(base + L::B_OFF + ch * 9 * L::B_TILE) + (uint64_t)((tap * L::B_TILE) >> 4);
                        } else {
                            sb = (int)(bcount % B_STAGES);
                            if (!mbar_wait_warp(bar_bfull + 8 * sb, (uint32_t)((bcount / B_STAGES) & 1), abort_flag, p.status, DT_W_B_FULL)) { ok = false; break; }
                            tc_fence_after();
                            b_desc0 = smem_desc_k128(base + L::B_OFF + sb * L::B_TILE);
                        }
                        const uint64_t a_desc = a_desc0 + (uint64_t)((((tap / 3) * DT_BOX_W + (tap % 3)) * 128) >> 4);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            if (tap == 0 && ks == 0)
                                { if (issuer) tc_mma<false>(d_tmem, a_desc, b_desc0, p.idesc, ch ? 1u : 0u); }
                            else
                                { if (issuer) tc_mma<false>(d_tmem, a_desc + (uint64_t)(ks * 2), b_desc0 + (uint64_t)(ks * 2), p.idesc, 1u); }
                        }
                        if (!B_RESIDENT) { if (issuer) tc_commit(bar_bempty + 8 * sb); ++bcount; }
                    }
                    if (!ok) break;
                    if (issuer) tc_commit(bar_aempty + 8 * st);
                    ++acount;
                }
                if (ok && issuer) tc_commit(bar_tfull + 8 * as);
                as ^= 1;
                if (as == 0) aphase ^= 1;
            }
        }
    } else {
        const int quarter = warp % 4;
        const int half = (warp - 2) / 4;              // which half of the BN filter columns this warp drains
        const int l = quarter * 32 + lane;            // accumulator lane = pixel of the tile: h = l / 8, w = l % 8
        const int ph_ = l / DT_TW, pw_ = l % DT_TW;
        constexpr int CHUNKS = BN / 64;               // 32-column chunks per warp
        int as = 0;
        uint32_t aphase = 0;
        bool ok = true;
        for (long long t = first; ok && t < total; t += step) {
            int n, ty, tx, nb;
            decode(t, n, ty, tx, nb);
            if (!mbar_wait_bounded(bar_tfull + 8 * as, aphase, abort_flag, p.status, DT_W_T_FULL)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int oy = ty * DT_TH + ph_, ox = tx * DT_TW + pw_;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * BN + half * (BN / 2));
            bool writer;
            long long pix;
            if (p.pool) {
                writer = ((ph_ | pw_) & 1) == 0 && (oy >> 1) < p.PH && (ox >> 1) < p.PW;
                pix = ((long long)n * p.PH + (oy >> 1)) * p.PW + (ox >> 1);
            } else {
                writer = oy < p.OH && ox < p.OW;
                pix = ((long long)n * p.OH + oy) * p.OW + ox;
            }
#pragma unroll 1
            for (int chunk = 0; chunk < CHUNKS; ++chunk) {
                uint32_t r[32];
                tmem_ld_32x32(lane_addr + chunk * 32, r);
                tmem_ld_wait();
                if (chunk == CHUNKS - 1) {
                    tc_fence_before();
                    mbar_arrive(bar_tempty + 8 * as);
                }
                const int k0 = nb * BN + half * (BN / 2) + chunk * 32;
                // bias + ReLU, packed to bf16 pairs; the 2x2 max is taken on the packed values (rounding is monotonic)
                uint32_t w[16];
#pragma unroll
                for (int e = 0; e < 32; e += 4) {
                    float4 b4 = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (p.bias && k0 + e + 4 <= p.K) b4 = __ldg(reinterpret_cast<const float4*>(p.bias + k0 + e));
                    float v0 = __uint_as_float(r[e]) + b4.x, v1 = __uint_as_float(r[e + 1]) + b4.y;
                    float v2 = __uint_as_float(r[e + 2]) + b4.z, v3 = __uint_as_float(r[e + 3]) + b4.w;
                    if (p.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); v2 = fmaxf(v2, 0.f); v3 = fmaxf(v3, 0.f); }
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(v0, v1), h1 = __floats2bfloat162_rn(v2, v3);
                    w[e / 2] = *reinterpret_cast<uint32_t*>(&h0);
                    w[e / 2 + 1] = *reinterpret_cast<uint32_t*>(&h1);
                }
                if (p.pool) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        uint32_t o = __shfl_xor_sync(0xffffffffu, w[e], 1);
                        __nv_bfloat162 m = __hmax2(*reinterpret_cast<__nv_bfloat162*>(&w[e]), *reinterpret_cast<__nv_bfloat162*>(&o));
                        uint32_t mu = *reinterpret_cast<uint32_t*>(&m);
                        o = __shfl_xor_sync(0xffffffffu, mu, 8);
                        m = __hmax2(m, *reinterpret_cast<__nv_bfloat162*>(&o));
                        w[e] = *reinterpret_cast<uint32_t*>(&m);
                    }
                }
                if (writer) {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.y) + pix * p.K + k0;
                    if (k0 + 32 <= p.K && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) reinterpret_cast<uint4*>(dst)[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e)
                            if (k0 + e < p.K) dst[e] = reinterpret_cast<const __nv_bfloat16*>(w)[e];
                    }
                }
            }
            as ^= 1;
            if (as == 0) aphase ^= 1;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * BN < 32 ? 32 : 2 * BN);
    }
}

// Filters for the kernel above: Wd[tap = 3r + s][k][Cp] = w[k][c][r][s] (any filter layout in, bf16), zero beyond C
template <typename T>
__global__ void pack_direct_tc_filters(const T* __restrict__ w, T* __restrict__ out, int K, int C, int Cp, Strides sw) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)9 * K * Cp) return;
    const int c = (int)(idx % Cp);
    const int k = (int)((idx / Cp) % K);
    const int tap = (int)(idx / ((long long)Cp * K));
    float v = c < C ? to_float<T>(w[k * sw.n + c * sw.c + (tap / 3) * sw.h + (tap % 3) * sw.w]) : 0.f;
    if (sizeof(T) == 4) v = from_float<tf32_t>(v).v;       // float filters are rounded to TF32 once, here
    out[idx] = from_float<T>(v);
}

template <int BN, int A_STAGES, int B_STAGES, bool B_RESIDENT>
int run(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const DtParams& p, cudaStream_t st) {
    using L = DtSmem<BN, A_STAGES, B_STAGES, B_RESIDENT>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA exceeded");
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(direct_tc_kernel<BN, A_STAGES, B_STAGES, B_RESIDENT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    WINO_CUDA_CHECK(attr_err);
    const long long total = (long long)p.N * p.tiles_x * p.tiles_y * p.nblocks;
    long long grid = total < sm_count() ? total : sm_count();
    if (B_RESIDENT) grid = grid / p.nblocks * p.nblocks;      // every CTA owns one filter block
    if (grid < 1) grid = p.nblocks;
    ProfScope prof(STAGE_DIRECT_TC, st);
    count_launch();
    direct_tc_kernel<BN, A_STAGES, B_STAGES, B_RESIDENT><<<(unsigned)grid, DT_THREADS, L::TOTAL, st>>>(tm_x, tm_w, p);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace

// 0: this shape never takes the direct kernel, 1: it always does, 2: it does for small batches only.  Does not look
// at d.n, so the format of the filter buffer (which follows this value) is the same for every batch size.
int direct_tc_mode(const wino_conv_desc& d) {
    static const int mode = [] { const char* e = getenv("WINO_DIRECT_TC"); return e ? atoi(e) : 1; }();
    if (mode == 0) return 0;
    // WINO_DIRECT_TC_MAXC forces the channel limit; by default the choice follows what was measured on B200 (batch 256):
    // up to 256 input channels the direct kernel beats the three-kernel Winograd pipeline (whose transform-domain
    // buffers are HBM-bound); at 512 channels Winograd's 4x fewer multiplies win, except on small images (14 x 14), on
    // a handful of images (fewer than 4 x 28 x 28 pixels in the batch), and where NCHW is involved.  512 -> 512 at 28 x 28,
    // direct / Winograd in microseconds: NHWC batch 4 27 / 18, 32 87 / 78, 64 161 / 145, 128 279 / 277 (float products;
    // 3-byte products from there on), 256 620 / 555; NCHW (x staged to NHWC, y stored NCHW by the direct kernel) batch 32
    // 95 / 128, 256 709 / 1060; CHWN batch 32 108 / 93, 256 752 / 688.
    static const int max_c = [] { const char* e = getenv("WINO_DIRECT_TC_MAXC"); return (e && *e) ? atoi(e) : -1; }();
    if (!(d.layout_in == WINO_NHWC && d.layout_out == WINO_NHWC && d.wino == 0) || out_type_differs(d)) return 0;
    if (d.dtype == WINO_TF32) {
        // float storage, TF32 operands: CTA-pair kernel only (32 channels per 128-byte chunk).  At half the tensor rate
        // of BF16 the direct kernel stays ahead of the Winograd pipeline up to 256 channels.
        if (!(d.c % 32 == 0 && direct_tc2_applies(d))) return 0;
        return (max_c >= 0 ? d.c <= max_c : d.c <= 256) ? 1 : 0;
    }
    if (!(d.dtype == WINO_BF16 && d.c % 64 == 0 && d.k % 8 == 0)) return 0;
    if (max_c >= 0) return d.c <= max_c ? 1 : 0;
    return (d.c <= 256 || (long long)d.h * d.w < 28 * 28) ? 1 : 2;
}

static bool handful_of_images(const wino_conv_desc& d) { return (long long)d.n * d.h * d.w < 4LL * 28 * 28; }

bool direct_tc_applies(const wino_conv_desc& d) {
    const int mode = direct_tc_mode(d);
    return mode == 1 || (mode == 2 && handful_of_images(d));
}

size_t direct_tc_filter_bytes(const wino_conv_desc& d) { return (size_t)9 * d.k * d.c * (d.dtype == WINO_BF16 ? 2 : 4); }

static wino_conv_desc nhwc_twin(const wino_conv_desc& d) {
    wino_conv_desc t = d;
    t.layout_in = WINO_NHWC; t.layout_out = WINO_NHWC;
    return t;
}

static bool via_nhwc_enabled(const wino_conv_desc& d) {
    static const bool off = [] { const char* e = getenv("WINO_DIRECT_RELAYOUT"); return e && e[0] == '0'; }();
    return !off && !(d.layout_in == WINO_NHWC && d.layout_out == WINO_NHWC);
}

bool direct_via_nhwc_applies(const wino_conv_desc& d) {
    if (!via_nhwc_enabled(d)) return false;
    const int mode = direct_tc_mode(nhwc_twin(d));
    // batch-dependent shapes: with NCHW on either side the staged direct kernel wins at every batch (see direct_tc_mode)
    return mode == 1 || (mode == 2 && (d.layout_in == WINO_NCHW || d.layout_out == WINO_NCHW || handful_of_images(d)));
}

int direct_filter_mode(const wino_conv_desc& d) {
    if (d.layout_in == WINO_NHWC && d.layout_out == WINO_NHWC) return direct_tc_mode(d);
    return via_nhwc_enabled(d) ? direct_tc_mode(nhwc_twin(d)) : 0;
}

static size_t round1k(size_t v) { return (v + 1023) & ~(size_t)1023; }

// the kernel behind the NHWC twin stores an NCHW result itself: no staging of y, no relayout pass after it
static bool y_stored_in_place(const wino_conv_desc& d) { return d.layout_out == WINO_NCHW && direct_tc_stores_nchw(nhwc_twin(d)); }

size_t direct_via_nhwc_staging_bytes(const wino_conv_desc& d, const Geometry& g) {
    const size_t es = d.dtype == WINO_BF16 ? 2 : 4;
    size_t need = 1024;
    if (d.layout_in != WINO_NHWC) need += round1k((size_t)d.n * d.c * d.h * d.w * es);
    if (d.layout_out != WINO_NHWC && !y_stored_in_place(d)) need += round1k((size_t)d.n * d.k * g.ph * g.pw * es);
    return need;
}

int launch_direct_via_nhwc(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                           void* scratch, size_t scratch_bytes, cudaStream_t st) {
    const size_t need = direct_via_nhwc_staging_bytes(d, g);
    if (!scratch || scratch_bytes < need)
        return fail(WINO_E_WORKSPACE, "conv forward: workspace of %zu bytes given, %zu needed (NHWC staging)", scratch_bytes, need);
    const int es = d.dtype == WINO_BF16 ? 2 : 4;
    uintptr_t p = ((uintptr_t)scratch + 1023) & ~(uintptr_t)1023;
    const void* xin = x;
    void* yout = y;
    int rc;
    if (d.layout_in != WINO_NHWC) {
        void* xs = (void*)p;
        p += round1k((size_t)d.n * d.c * d.h * d.w * es);
        if ((rc = launch_relayout(d.layout_in, WINO_NHWC, d.n, d.c, d.h, d.w, es, x, xs, st))) return rc;
        xin = xs;
    }
    const bool in_place = y_stored_in_place(d);
    if (d.layout_out != WINO_NHWC && !in_place) yout = (void*)p;
    const wino_conv_desc t = nhwc_twin(d);
    if ((rc = launch_direct_tc(t, g, xin, packed, bias, yout, st, in_place))) return rc;
    if (d.layout_out != WINO_NHWC && !in_place) return launch_relayout(WINO_NHWC, d.layout_out, d.n, d.k, g.ph, g.pw, es, yout, y, st);
    return WINO_OK;
}

int launch_direct_tc_pack(const wino_conv_desc& d, const void* w, void* packed, cudaStream_t st) {
    const long long total = (long long)9 * d.k * d.c;
    ProfScope prof(STAGE_FILTER, st);
    count_launch();
    if (d.dtype == WINO_TF32)
        pack_direct_tc_filters<float><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const float*)w, (float*)packed, d.k, d.c, d.c,
                                                                                     filter_strides(d.layout_in, d.k, d.c));
    else
        pack_direct_tc_filters<__nv_bfloat16><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
            (const __nv_bfloat16*)w, (__nv_bfloat16*)packed, d.k, d.c, d.c, filter_strides(d.layout_in, d.k, d.c));
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

int launch_direct_tc(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                     cudaStream_t st, bool y_nchw) {
    if (d.n == 0) return WINO_OK;
    if (direct_tc2_applies(d)) return launch_direct_tc2(d, g, x, packed, bias, y, st, y_nchw);
    if (y_nchw) return fail(WINO_E_UNSUPPORTED, "direct conv: the single-CTA kernel stores NHWC only");
    if (((uintptr_t)x | (uintptr_t)packed | (uintptr_t)y | (d.has_bias ? (uintptr_t)bias : 0)) & 15)
        return fail(WINO_E_BADARG, "direct conv: buffers (and the bias) must be 16-byte aligned");
    DtParams p;
    p.bias = d.has_bias ? bias : nullptr; p.y = y;
    p.N = d.n; p.OH = g.oh; p.OW = g.ow; p.K = d.k; p.pad = d.pad; p.PH = g.ph; p.PW = g.pw;
    p.tiles_x = (g.ow + DT_TW - 1) / DT_TW; p.tiles_y = (g.oh + DT_TH - 1) / DT_TH;
    p.cchunks = d.c / 64;
    p.relu = d.relu; p.pool = d.pool2x2; p.y_nchw = 0;
    int rc = status_word(&p.status);
    if (rc) return rc;
    const int bn = d.k >= 128 ? 128 : 64;
    p.nblocks = (d.k + bn - 1) / bn;
    p.idesc = make_idesc(OP_BF16, bn);
    CUtensorMap tm_x, tm_w;
    {
        const unsigned long long dims[4] = {(unsigned long long)d.c, (unsigned long long)d.w, (unsigned long long)d.h, (unsigned long long)d.n};
        const unsigned long long strides[3] = {d.c * 2ull, (unsigned long long)d.w * d.c * 2ull, (unsigned long long)d.h * d.w * d.c * 2ull};
        const unsigned box[4] = {64u, (unsigned)DT_BOX_W, (unsigned)DT_BOX_H, 1u};
        if ((rc = encode_tensor_map(&tm_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x, dims, strides, box, true))) return rc;
    }
    if ((rc = make_map_k128(&tm_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, packed, d.c, d.k, d.k, 9, bn))) return rc;
    // filters stay resident in shared memory when the layer has a single 64-channel chunk (C = 64)
    const bool resident = p.cchunks == 1;
    if (bn == 64) return resident ? run<64, 6, 2, true>(tm_x, tm_w, p, st) : run<64, 6, 6, false>(tm_x, tm_w, p, st);
    return resident ? run<128, 3, 2, true>(tm_x, tm_w, p, st) : run<128, 6, 4, false>(tm_x, tm_w, p, st);
}

}  // namespace wino

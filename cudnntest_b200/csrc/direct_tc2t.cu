// Direct (implicit-GEMM) 3x3 convolution on CTA pairs with the FILTERS as the M operand, for layers with at least 256
// filters (NHWC, BF16 or TF32 operands), sm_100a.
//
// direct_tc2.cu makes the pixels the 128 accumulator rows of a CTA, which fixes the pixel tile at 8 x 16 and wastes
// MMA rows on images whose height is not a multiple of 16 (56, 28, 14: 12.5 - 30 %).  Here the roles are swapped:
//   * D[filter][pixel]: each CTA of a pair owns 128 of the pair's 256 filters (its accumulator lanes) and one pixel
//     tile of 8 x TH pixels; the pair's MMA (tcgen05.mma.cta_group::2, M = 256) has N = 2 * 8 * TH pixel columns, and
//     N only has to be a multiple of 16, so TH = 14 fits 56, 28 and 14 exactly (TH is picked per layer from
//     8, 10, 12, 14, 16);
//   * the pixel operand is the same 128-byte-swizzled halo box as in direct_tc2.cu (10 x (TH + 2) pixels, one 4-D TMA
//     load per 64-channel chunk, nine taps through shifted descriptors, 8-pixel row groups 1280 bytes apart), now
//     read as the N-side operand whose rows are split between the two CTAs: each CTA loads and holds its own box;
//   * the filter operand is a plain 128-row K-major tile per tap and chunk, streamed through a TMA ring;
//   * epilogue: a thread owns one filter (accumulator lane) and reads the pixels of one of the pair's two tiles from
//     tensor memory, 16 columns (two pixel rows) at a time, the next load in flight while a step's values leave.  The
//     bias is one scalar per thread, the 2x2 max-pool is taken inside the thread's registers, and a warp's 32 lanes
//     store 32 consecutive NHWC channels of a pixel (64 contiguous bytes for BF16); without pooling neighbouring
//     lanes first exchange a packed word, so that each stores both filters of one pixel row as one 4- or 8-byte
//     word.  The drain runs underneath the MMAs of the other accumulator stage.
// What bounds it: the shared-memory fill.  Every 64-channel chunk brings 9 x 16 KB of filter taps and a 20 KB halo box
// into each CTA for 128 x 224 x 576 multiply-adds, which at the full tensor rate is more than the L2 delivers to 148 SMs;
// tensor memory (512 columns, half of them draining) caps the pixels one filter load serves at 224.
// Barrier protocol, bounded waits and the final cluster barrier are those of direct_tc2.cu.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"
#include "direct_tc.cuh"

namespace wino {

namespace {

constexpr int DTT_W_TILE = 128 * 128;         // one tap of one chunk for this CTA's 128 filters

// Stores CNT (4 or 8) consecutive outputs of one row of an NCHW plane, of which the first `left` lie inside the row
// (pitch = row length in elements).  The element offset `off` and the pitch decide the alignment: groups of G elements
// go out as one vector when both are multiples of G (up to 16 bytes), single elements otherwise.
template <bool F32, int CNT>
__device__ __forceinline__ void store_row_nchw(void* y, long long off, const float* v, int left, int pitch) {
    const int align = (int)((off | (long long)pitch) & 7);
    if (F32) {
        float* dst = reinterpret_cast<float*>(y) + off;
        const bool vec4 = (align & 3) == 0;
#pragma unroll
        for (int e = 0; e < CNT; e += 4) {
            if (vec4 && e + 4 <= left) {
                *reinterpret_cast<float4*>(dst + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (e + i < left) dst[e + i] = v[e + i];
            }
        }
    } else {
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(y) + off;
        uint32_t w[CNT / 2];
#pragma unroll
        for (int e = 0; e < CNT / 2; ++e) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
            w[e] = *reinterpret_cast<uint32_t*>(&h);
        }
        if (CNT == 8 && align == 0 && left >= 8) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2 % (CNT / 2)], w[3 % (CNT / 2)]);
            return;
        }
        const bool vec4 = (align & 3) == 0, vec2 = (align & 1) == 0;
#pragma unroll
        for (int e = 0; e < CNT; e += 4) {
            if (vec4 && e + 4 <= left) {
                *reinterpret_cast<uint2*>(dst + e) = make_uint2(w[e / 2], w[e / 2 + 1]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; i += 2) {
                    if (vec2 && e + i + 2 <= left) {
                        *reinterpret_cast<uint32_t*>(dst + e + i) = w[(e + i) / 2];
                    } else {
                        if (e + i < left) dst[e + i] = __float2bfloat16_rn(v[e + i]);
                        if (e + i + 1 < left) dst[e + i + 1] = __float2bfloat16_rn(v[e + i + 1]);
                    }
                }
            }
        }
    }
}

// FLATW = 0: a pixel tile is 8 columns x TH rows of the image and the halo box 10 x (TH + 2) pixels.
// FLATW > 0 (images exactly FLATW - 2 pixels wide): a tile is TH whole image rows.  The halo box is FLATW x (TH + 2)
// pixels, and the MMA's pixel index runs over the box row after row: index j = row * FLATW + column, tap (dy, dx) reads
// pixel j + dy * FLATW + dx, which is a plain shift of the start address.  The two indices per row that fall on the halo
// columns are computed and dropped.  28-wide images lose 6.7 % of the MMA columns that way instead of the 12.5 % of
// four 8-wide tiles, and a filter tap loaded from the L2 serves 224 real pixels of a pair instead of 196.
template <int TH, int A_STAGES, int B_STAGES, int FLATW = 0>
struct DttSmem {
    static constexpr int BOX_W = FLATW ? FLATW : DT_BOX_W;
    static constexpr int PX_BYTES = BOX_W * (TH + 2) * 128;                    // bytes one halo box brings in
    // (the last taps of a flat tile read two pixels past the box: they only feed dropped columns, and stay inside the slot)
    static constexpr int PX_STRIDE = (PX_BYTES + 256 + 1023) / 1024 * 1024;
    static constexpr int A_OFF = 0;                                            // pixel boxes
    static constexpr int B_OFF = A_OFF + A_STAGES * PX_STRIDE;                 // filter taps
    static constexpr int BAR_OFF = B_OFF + B_STAGES * DTT_W_TILE;
    static constexpr int NPIX = FLATW ? FLATW * TH : DT_TW * TH;               // pixel columns per CTA
    static constexpr int NCOL = 2 * NPIX;                                      // MMA N: both CTAs' pixels
    static constexpr int ACC = 512 / NCOL < 4 ? 512 / NCOL : 4;
    static constexpr int NBARS = 2 * A_STAGES + 2 * B_STAGES + 2 * ACC;
    static constexpr int SLOT_OFF = BAR_OFF + 8 * NBARS;
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;
};

template <int TH, int A_STAGES, int B_STAGES, bool TF32, int FLATW = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(DT_THREADS, 1)
direct_tc2t_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const DtParams p) {
    using L = DttSmem<TH, A_STAGES, B_STAGES, FLATW>;
    static_assert(FLATW ? (TH == 4 && FLATW == 30) : (TH % 2 == 0 && TH >= 8 && TH <= 16), "pixel tile shape");
    static_assert(L::NPIX % 8 == 0 && L::NPIX <= 128, "pixel columns per CTA");
    static_assert(L::ACC >= 2, "accumulators are at least double-buffered");
    constexpr int ACC = L::ACC, NPIX = L::NPIX, NCOL = L::NCOL;
    constexpr int CPC = TF32 ? 32 : 64;      // channels per 128-byte chunk
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;      // same offset in both CTAs of the pair
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFF;
    const uint32_t bar_afull = bars, bar_aempty = bar_afull + 8 * A_STAGES;
    const uint32_t bar_bfull = bar_aempty + 8 * A_STAGES, bar_bempty = bar_bfull + 8 * B_STAGES;
    const uint32_t bar_tfull = bar_bempty + 8 * B_STAGES, bar_tempty = bar_tfull + 8 * ACC;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::SLOT_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::SLOT_OFF + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs, owns the "full" barriers)
    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; ++s) { mbar_init(bar_afull + 8 * s, 1); mbar_init(bar_aempty + 8 * s, 1); }
        for (int s = 0; s < B_STAGES; ++s) { mbar_init(bar_bfull + 8 * s, 1); mbar_init(bar_bempty + 8 * s, 1); }
        for (int a = 0; a < ACC; ++a) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 2 * DT_EPI_WARPS); }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), 512);
    tc_fence_before();
    cluster_sync_all();            // barriers of both CTAs initialised before any remote arrive or TMA completion
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();                    // everything above overlapped the previous kernel's last wave; tensors are touched from here on

    const long long tiles_img = (long long)p.tiles_x * p.tiles_y;
    const long long total_tiles = (long long)p.N * tiles_img;
    const long long ngroups = (total_tiles + 1) / 2;                  // a pair takes two consecutive pixel tiles
    const long long total = ngroups * p.nblocks;
    const long long pair = blockIdx.x / 2, npairs = gridDim.x / 2;

    // work item -> 256-filter block and the pixel tile of CTA `who` of the pair (clamped to the last tile when the
    // batch runs out: the duplicate is computed and not stored)
    auto decode = [&](long long u, uint32_t who, int& n, int& ty, int& tx, int& nb, bool& valid) {
        nb = (int)(u % p.nblocks);
        long long tl = (u / p.nblocks) * 2 + who;
        valid = tl < total_tiles;
        if (!valid) tl = total_tiles - 1;
        tx = (int)(tl % p.tiles_x); tl /= p.tiles_x;
        ty = (int)(tl % p.tiles_y);
        n = (int)(tl / p.tiles_y);
    };

    if (warp == 0) {
        {   // the whole warp walks the rings (warp-uniform addresses); one elected lane issues the copies
            const bool issuer = elect_one();
            bool ok = true;
            unsigned long long acount = 0, bcount = 0;
            for (long long u = pair; ok && u < total; u += npairs) {
                int n, ty, tx, nb; bool valid;
                decode(u, rank, n, ty, tx, nb, valid);
                for (int ch = 0; ok && ch < p.cchunks; ++ch) {
                    const int st = (int)(acount % A_STAGES);
                    if (!mbar_wait_warp(bar_aempty + 8 * st, (uint32_t)(((acount / A_STAGES) & 1) ^ 1), abort_flag, p.status, DT_W_A_EMPTY)) { ok = false; break; }
                    if (rank == 0 && issuer) mbar_arrive_expect_tx(bar_afull + 8 * st, 2 * L::PX_BYTES);
                    if (issuer) tma_load_4d_pair(base + L::A_OFF + st * L::PX_STRIDE, &tm_x, mapa_shared(bar_afull + 8 * st, 0), ch * CPC,
                                                 tx * DT_TW - p.pad, ty * TH - p.pad, n);
                    ++acount;
                    for (int tap = 0; tap < 9; ++tap) {
                        const int sb = (int)(bcount % B_STAGES);
                        if (!mbar_wait_warp(bar_bempty + 8 * sb, (uint32_t)(((bcount / B_STAGES) & 1) ^ 1), abort_flag, p.status, DT_W_B_EMPTY)) { ok = false; break; }
                        if (rank == 0 && issuer) mbar_arrive_expect_tx(bar_bfull + 8 * sb, 2 * DTT_W_TILE);
                        if (issuer) tma_load_3d_pair(base + L::B_OFF + sb * DTT_W_TILE, &tm_w, mapa_shared(bar_bfull + 8 * sb, 0), ch * CPC,
                                                     nb * 256 + (int)rank * 128, tap);
                        ++bcount;
                    }
                }
            }
            if (!ok && issuer) drain_after_abort();
        }
    } else if (warp == 1) {
        // MMA issue (leader CTA only): warp-uniform loop, one elected lane issues the tcgen05 instructions
        if (rank == 0) {
            const bool issuer = elect_one();
            bool ok = true;
            unsigned long long acount = 0, bcount = 0;
            int as = 0;
            uint32_t aphase = 0;
            for (long long u = pair; ok && u < total; u += npairs) {
                if (!mbar_wait_warp(bar_tempty + 8 * as, aphase ^ 1, abort_flag, p.status, DT_W_T_EMPTY)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * NCOL);
                for (int ch = 0; ok && ch < p.cchunks; ++ch) {
                    const int st = (int)(acount % A_STAGES);
                    if (!mbar_wait_warp(bar_afull + 8 * st, (uint32_t)((acount / A_STAGES) & 1), abort_flag, p.status, DT_W_A_FULL)) { ok = false; break; }
                    tc_fence_after();
                    // 8-pixel groups of the N operand: one tile row (next group = next halo row), or consecutive pixels of the box
                    const uint64_t px_desc0 = smem_desc_k128_sbo(base + L::A_OFF + st * L::PX_STRIDE, FLATW ? 1024 : DT_BOX_W * 128);
#pragma unroll
                    for (int tap = 0; tap < 9; ++tap) {
                        const int sb = (int)(bcount % B_STAGES);
                        if (!mbar_wait_warp(bar_bfull + 8 * sb, (uint32_t)((bcount / B_STAGES) & 1), abort_flag, p.status, DT_W_B_FULL)) { ok = false; break; }
                        tc_fence_after();
                        const uint64_t w_desc = smem_desc_k128(base + L::B_OFF + sb * DTT_W_TILE);
                        const uint64_t px_desc = px_desc0 + (uint64_t)((((tap / 3) * L::BOX_W + (tap % 3)) * 128) >> 4);
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            if (tap == 0 && ks == 0)
                                { if (issuer) tc_mma_pair<TF32>(d_tmem, w_desc, px_desc, p.idesc, ch ? 1u : 0u); }
                            else
                                { if (issuer) tc_mma_pair<TF32>(d_tmem, w_desc + (uint64_t)(ks * 2), px_desc + (uint64_t)(ks * 2), p.idesc, 1u); }
                        }
                        if (issuer) tc_commit_pair(bar_bempty + 8 * sb, 3);
                        ++bcount;
                    }
                    if (!ok) break;
                    if (issuer) tc_commit_pair(bar_aempty + 8 * st, 3);
                    ++acount;
                }
                if (ok && issuer) tc_commit_pair(bar_tfull + 8 * as, 3);
                if (++as == ACC) { as = 0; aphase ^= 1; }
            }
        }
    } else {
        const int quarter = warp % 4;                 // accumulator lanes [32 quarter, 32 quarter + 32) = 32 filters
        const uint32_t who = (uint32_t)((warp - 2) / 4);   // which of the pair's two pixel tiles this warp drains
        const uint32_t tempty_leader0 = mapa_shared(bar_tempty, 0);
        int as = 0;
        uint32_t aphase = 0;
        bool ok = true;
        for (long long u = pair; ok && u < total; u += npairs) {
            if (!mbar_wait_bounded(bar_tfull + 8 * as, aphase, abort_flag, p.status, DT_W_T_FULL)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            int n, ty, tx, nb; bool valid;
            decode(u, who, n, ty, tx, nb, valid);
            const int kch = nb * 256 + (int)rank * 128 + quarter * 32 + lane;      // this thread's filter
            const bool k_ok = valid && kch < p.K;
            const float bias = (p.bias && kch < p.K) ? __ldg(p.bias + kch) : 0.f;
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * NCOL) + who * NPIX;
            const int oy0 = ty * TH;
            // lanes 2j and 2j+1 hold neighbouring filters: in the unpooled NHWC store the even lane takes the upper pixel
            // row of a step for both filters and the odd lane the lower one, so that every store is one 4- or 8-byte word
            const int odd = lane & 1;
            // bias, ReLU, pool and store of 8 pixels x 2 rows of this thread's filter: v[e] = (row oy, column ox0 + e),
            // v[8 + e] = (row oy + 1, column ox0 + e)
            auto emit = [&](float (&v)[16], int oy, int ox0) {
                const int nvalid = min(8, p.OW - ox0);
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    v[e] += bias;
                    if (p.relu) v[e] = fmaxf(v[e], 0.f);
                }
                if (p.y_nchw) {
                    // NCHW: this thread's filter is a plane of y and its registers are runs of consecutive pixels of a row
                    // (8 outputs, or 4 pooled ones): they leave as the widest vectors the row pitch keeps aligned
                    if (k_ok) {
                        if (p.pool) {
                            const int py = oy >> 1;
                            if (py < p.PH) {
                                float m[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) m[q] = fmaxf(fmaxf(v[2 * q], v[2 * q + 1]), fmaxf(v[8 + 2 * q], v[8 + 2 * q + 1]));
                                store_row_nchw<TF32, 4>(p.y, (((long long)n * p.K + kch) * p.PH + py) * p.PW + (ox0 >> 1), m, p.PW - (ox0 >> 1), p.PW);
                            }
                        } else {
#pragma unroll
                            for (int rr = 0; rr < 2; ++rr)
                                if (oy + rr < p.OH)
                                    store_row_nchw<TF32, 8>(p.y, (((long long)n * p.K + kch) * p.OH + oy + rr) * p.OW + ox0, v + 8 * rr, p.OW - ox0, p.OW);
                        }
                    }
                } else if (p.pool) {
                    const int py = oy >> 1;
                    if (k_ok && py < p.PH) {
                        // element offset of the first pooled pixel of this row of windows; the others are K apart
                        const long long o0 = (((long long)n * p.PH + py) * p.PW + (ox0 >> 1)) * p.K + kch;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if ((ox0 >> 1) + q < p.PW) {
                                const float m = fmaxf(fmaxf(v[2 * q], v[2 * q + 1]), fmaxf(v[8 + 2 * q], v[8 + 2 * q + 1]));
                                if (TF32) reinterpret_cast<float*>(p.y)[o0 + q * p.K] = m;
                                else reinterpret_cast<__nv_bfloat16*>(p.y)[o0 + q * p.K] = __float2bfloat16_rn(m);
                            }
                        }
                    }
                } else {
                    // K is a multiple of 16: both lanes of a pair are inside K together, and the shuffles run on every lane
                    const int row = oy + odd;
                    const bool st_ok = k_ok && row < p.OH;
                    const long long o0 = (((long long)n * p.OH + row) * p.OW + ox0) * p.K + (kch & ~1);
                    if (TF32) {
                        float* dst = reinterpret_cast<float*>(p.y) + o0;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float keep = odd ? v[8 + e] : v[e];
                            const float recv = __shfl_xor_sync(0xffffffffu, odd ? v[e] : v[8 + e], 1);
                            if (st_ok && e < nvalid)
                                *reinterpret_cast<float2*>(dst + (long long)e * p.K) = odd ? make_float2(recv, keep) : make_float2(keep, recv);
                        }
                    } else {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.y) + o0;
                        const uint32_t sel = odd ? 0x3276u : 0x5410u;
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const __nv_bfloat162 both = __floats2bfloat162_rn(v[e], v[8 + e]);     // low half: upper row
                            const uint32_t own = *reinterpret_cast<const uint32_t*>(&both);
                            const uint32_t recv = __shfl_xor_sync(0xffffffffu, own, 1);
                            if (st_ok && e < nvalid)
                                *reinterpret_cast<uint32_t*>(dst + (long long)e * p.K) = __byte_perm(own, recv, sel);
                        }
                    }
                }
            };
            if constexpr (FLATW != 0) {
                // TH = 4 rows of FLATW = 30 columns: a pair of rows is 60 consecutive accumulator columns, read as 64 from a
                // multiple of 8 (0 for rows 0-1, 56 for rows 2-3: their first column is then register 4)
#pragma unroll
                for (int rp = 0; rp < 2; ++rp) {
                    constexpr int OW_ = FLATW - 2;
                    uint32_t r[64];
                    tmem_ld_32x32(lane_addr + rp * 56, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                    tmem_ld_32x32(lane_addr + rp * 56 + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                    tmem_ld_wait();
                    if (rp == 1) {                        // accumulator stage drained: release it on the leader
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * as);
                    }
                    const int off = rp * 4;
#pragma unroll
                    for (int c0 = 0; c0 < OW_; c0 += 8) {
                        float v[16];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            // columns past the image (the last group has 4) are never stored: any register will do
                            const int c = c0 + e < OW_ ? c0 + e : OW_ - 1;
                            v[e] = __uint_as_float(r[off + c]);
                            v[8 + e] = __uint_as_float(r[off + FLATW + c]);
                        }
                        emit(v, oy0 + 2 * rp, c0);
                    }
                }
            } else {
                const int ox0 = tx * DT_TW;
                uint32_t r[16];
                tmem_ld_32x16(lane_addr, r);
#pragma unroll 1
                for (int pr = 0; pr < TH / 2; ++pr) {     // two pixel rows (16 columns) per step: one row of 2x2 pool windows
                    tmem_ld_wait();
                    float v[16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] = __uint_as_float(r[e]);
                    if (pr == TH / 2 - 1) {               // accumulator stage drained: release it on the leader
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * as);
                    } else {
                        tmem_ld_32x16(lane_addr + (pr + 1) * 16, r);    // in flight while this step's values leave
                    }
                    emit(v, oy0 + 2 * pr, ox0);
                }
            }
            if (++as == ACC) { as = 0; aphase ^= 1; }
        }
    }

    // neither CTA may leave (or give back tensor memory) while its partner can still read its shared memory,
    // signal its barriers or run an MMA over both tensor memories
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

template <int TH, int A_STAGES, int B_STAGES, bool TF32, int FLATW = 0>
int run_t(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const DtParams& p, cudaStream_t st) {
    using L = DttSmem<TH, A_STAGES, B_STAGES, FLATW>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA exceeded");
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(direct_tc2t_kernel<TH, A_STAGES, B_STAGES, TF32, FLATW>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    WINO_CUDA_CHECK(attr_err);
    const long long total_tiles = (long long)p.N * p.tiles_x * p.tiles_y;
    const long long total = (total_tiles + 1) / 2 * p.nblocks;
    long long pairs = sm_count() / 2;
    if (total < pairs) pairs = total;
    if (pairs < 1) pairs = 1;
    ProfScope prof(STAGE_DIRECT_TC, st);
    count_launch();
    WINO_CUDA_CHECK(launch_kernel(direct_tc2t_kernel<TH, A_STAGES, B_STAGES, TF32, FLATW>, dim3((unsigned)(2 * pairs)), dim3(DT_THREADS), L::TOTAL, st,
                                  pdl_enabled(), tm_x, tm_w, p));
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

template <int TH>
int run_th(bool tf32, const CUtensorMap& tm_x, const CUtensorMap& tm_w, const DtParams& p, cudaStream_t st) {
    return tf32 ? run_t<TH, 4, 8, true>(tm_x, tm_w, p, st) : run_t<TH, 4, 8, false>(tm_x, tm_w, p, st);
}

// pixel tile height in {16, 14, 12, 10, 8} that wastes the fewest rows of an image oh rows high (the taller on ties)
int pick_tile_height(int oh) {
    int best = 16;
    long long best_rows = (long long)((oh + 15) / 16) * 16;
    for (int th = 14; th >= 8; th -= 2) {
        const long long rows = (long long)((oh + th - 1) / th) * th;
        if (rows < best_rows) { best_rows = rows; best = th; }
    }
    return best;
}

}  // namespace

bool direct_tc2t_applies(const wino_conv_desc& d) {
    static const bool off = [] { const char* e = getenv("WINO_DIRECT_TC_T"); return e && e[0] == '0'; }();
    return !off && direct_tc2_applies(d) && d.k >= 256 && d.k % 128 == 0;
}

int launch_direct_tc2t(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                       cudaStream_t st, bool y_nchw) {
    if (d.n == 0) return WINO_OK;
    if (((uintptr_t)x | (uintptr_t)packed | (uintptr_t)y | (d.has_bias ? (uintptr_t)bias : 0)) & 15)
        return fail(WINO_E_BADARG, "direct conv: buffers (and the bias) must be 16-byte aligned");
    const bool tf32 = d.dtype == WINO_TF32;
    const int es = tf32 ? 4 : 2;
    // 28-wide images: tiles of 4 whole rows over the flattened halo box (see DttSmem); WINO_DIRECT_FLAT=0 keeps the 8-wide tiles
    static const bool flat_off = [] { const char* e = getenv("WINO_DIRECT_FLAT"); return e && e[0] == '0'; }();
    const bool flat = !flat_off && g.ow == 28;
    const int th = flat ? 4 : pick_tile_height(g.oh);
    const int box_w = flat ? 30 : DT_BOX_W, npix = flat ? 30 * 4 : DT_TW * th;
    DtParams p;
    p.bias = d.has_bias ? bias : nullptr; p.y = y;
    p.N = d.n; p.OH = g.oh; p.OW = g.ow; p.K = d.k; p.pad = d.pad; p.PH = g.ph; p.PW = g.pw;
    p.tiles_x = flat ? 1 : (g.ow + DT_TW - 1) / DT_TW; p.tiles_y = (g.oh + th - 1) / th;
    p.cchunks = d.c / (128 / es);
    p.relu = d.relu; p.pool = d.pool2x2; p.y_nchw = y_nchw ? 1 : 0;
    p.nblocks = (d.k + 255) / 256;
    p.idesc = make_idesc(tf32 ? OP_TF32 : OP_BF16, 2 * npix, 256);
    int rc = status_word(&p.status);
    if (rc) return rc;
    CUtensorMap tm_x, tm_w;
    {
        const unsigned long long ues = (unsigned long long)es;
        const unsigned long long dims[4] = {(unsigned long long)d.c, (unsigned long long)d.w, (unsigned long long)d.h, (unsigned long long)d.n};
        const unsigned long long strides[3] = {d.c * ues, (unsigned long long)d.w * d.c * ues, (unsigned long long)d.h * d.w * d.c * ues};
        const unsigned box[4] = {(unsigned)(128 / es), (unsigned)box_w, (unsigned)(th + 2), 1u};
        if ((rc = encode_tensor_map(&tm_x, tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x, dims, strides, box, true))) return rc;
    }
    if ((rc = make_map_k128(&tm_w, tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, es, packed, d.c, d.k, d.k, 9, 128))) return rc;
    if (flat) return tf32 ? run_t<4, 4, 8, true, 30>(tm_x, tm_w, p, st) : run_t<4, 4, 8, false, 30>(tm_x, tm_w, p, st);
    switch (th) {
        case 16: return run_th<16>(tf32, tm_x, tm_w, p, st);
        case 14: return run_th<14>(tf32, tm_x, tm_w, p, st);
        case 12: return run_th<12>(tf32, tm_x, tm_w, p, st);
        case 10: return run_th<10>(tf32, tm_x, tm_w, p, st);
        default: return run_th<8>(tf32, tm_x, tm_w, p, st);
    }
}

}  // namespace wino

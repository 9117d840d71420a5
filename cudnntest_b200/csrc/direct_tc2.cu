// Direct (implicit-GEMM) 3x3 convolution on tcgen05 with CTA pairs (cta_group::2) for NHWC BF16 layers, sm_100a.
//
// Same data flow as direct_tc.cu (one 4-D TMA halo box per 8 x 16 pixel tile and 64-channel chunk, nine filter taps
// read through shifted shared-memory descriptors), but two CTAs of a cluster work as one MMA unit:
//   * each CTA owns MT pixel tiles (its 128 accumulator lanes per tile) and HALF of the BN filter rows of every tap;
//     one tcgen05.mma.cta_group::2 issued by the leader CTA multiplies the pair's 256 pixels by all BN filters, reading
//     each CTA's pixels and each CTA's half of the filters from that CTA's shared memory.  Per MMA a CTA therefore
//     reads BN/2 instead of BN filter rows from shared memory and loads half of the filter bytes from L2: with a
//     single CTA the 128 x 64 and 128 x 128 MMA shapes are bound by shared-memory operand reads, not by the tensor pipe;
//   * both CTAs load their own boxes and filter halves with TMA (no multicast); the bytes are counted on the
//     leader's "full" mbarriers, the leader's tcgen05.commit frees ring slots and publishes accumulators in both
//     CTAs at once, epilogue warps of both CTAs release the accumulator stage on the leader's barrier;
//   * accumulators rotate through up to four tensor-memory stages (short reduction loops leave little time per
//     stage and the release crosses the cluster);
//   * with MT = 2 a filter tap loaded once serves two pixel tiles per CTA (four per pair), halving the L2 -> shared
//     filter traffic per flop again.
// Every wait is bounded (2 s) and reports to the device status word; both CTAs meet at a cluster barrier before
// tensor memory is released, so neither leaves while the other can still touch its shared memory or barriers.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"
#include "direct_tc.cuh"

namespace wino {

namespace {

// 2x2 max-pool across the lanes of a warp whose lane index is 8 * (pixel row) + (pixel column) of a tile.  A full
// butterfly (every lane exchanges every word with lane ^ 1, then lane ^ 8) costs two shuffles per word and leaves the
// same result in four lanes; here each exchange also halves what a lane keeps: the odd column keeps the upper half of
// the words, the odd row the upper half of what is left.  3/4 of a shuffle per word, and every lane ends with
// WORDS / 4 results: words [first, first + WORDS / 4) of the window's pooled values, first = pooled_first_word().
// Shuffles share the shared-memory data path with the MMA's operand reads, which is what this kernel is short of.
template <int WORDS, typename Op>
__device__ __forceinline__ void pool2x2_split(uint32_t (&w)[WORDS], int lane, Op op) {
    constexpr int H = WORDS / 2, Q = WORDS / 4;
    const bool oddx = lane & 1, oddy = lane & 8;
#pragma unroll
    for (int i = 0; i < H; ++i) {
        const uint32_t keep = oddx ? w[H + i] : w[i];
        const uint32_t got = __shfl_xor_sync(0xffffffffu, oddx ? w[i] : w[H + i], 1);
        w[i] = op(keep, got);
    }
#pragma unroll
    for (int i = 0; i < Q; ++i) {
        const uint32_t keep = oddy ? w[Q + i] : w[i];
        const uint32_t got = __shfl_xor_sync(0xffffffffu, oddy ? w[i] : w[Q + i], 8);
        w[i] = op(keep, got);
    }
}
template <int WORDS>
__device__ __forceinline__ int pooled_first_word(int lane) { return ((lane & 1) ? WORDS / 2 : 0) + ((lane & 8) ? WORDS / 4 : 0); }

template <int BN, int MT, int A_STAGES, int B_STAGES, bool B_RESIDENT, int RES_CHUNKS, bool STG = false>
struct Dt2Smem {
    static constexpr int B_TILE = (BN / 2) * 128;          // this CTA's half of one tap of one 64-channel chunk
    static constexpr int A_OFF = 0;
    static constexpr int B_OFF = A_OFF + A_STAGES * DT_A_STRIDE;
    static constexpr int B_BYTES = (B_RESIDENT ? 9 * RES_CHUNKS : B_STAGES) * B_TILE;
    static constexpr int STG_OFF = B_OFF + B_BYTES;        // optional store staging: 4 KiB per epilogue warp
    static constexpr int BAR_OFF = STG_OFF + (STG ? DT_EPI_WARPS * 4096 : 0);
    static constexpr int TMEM_COLS = 512;                  // the whole tensor memory: one CTA per SM anyway
    static constexpr int ACC = TMEM_COLS / (MT * BN) < 4 ? TMEM_COLS / (MT * BN) : 4;   // accumulator stages
    static constexpr int NBARS = 2 * A_STAGES + 2 * B_STAGES + 2 * ACC + 1;
    static constexpr int SLOT_OFF = BAR_OFF + 8 * NBARS;
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;
};

template <int BN, int MT, int A_STAGES, int B_STAGES, bool B_RESIDENT, int RES_CHUNKS, bool TF32, bool STG = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(DT_THREADS, 1)
direct_tc2_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w,
                  const __grid_constant__ CUtensorMap tm_y, const DtParams p) {
    using L = Dt2Smem<BN, MT, A_STAGES, B_STAGES, B_RESIDENT, RES_CHUNKS, STG>;
    static_assert(!STG || (BN == 128 && !TF32), "store staging exists for 128-filter blocks of bf16 outputs");
    static_assert(L::ACC >= 2, "accumulators are at least double-buffered");
    constexpr int ACC = L::ACC;
    constexpr int CPC = TF32 ? 32 : 64;      // channels per 128-byte chunk
    static_assert(A_STAGES >= MT, "one work item needs MT boxes in flight");
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;      // same offset in both CTAs of the pair
    uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFF;
    const uint32_t bar_afull = bars, bar_aempty = bar_afull + 8 * A_STAGES;
    const uint32_t bar_bfull = bar_aempty + 8 * A_STAGES, bar_bempty = bar_bfull + 8 * B_STAGES;
    const uint32_t bar_tfull = bar_bempty + 8 * B_STAGES, bar_tempty = bar_tfull + 8 * ACC, bar_bres = bar_tempty + 8 * ACC;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::SLOT_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::SLOT_OFF + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs, owns the "full" barriers)
    if (threadIdx.x == 0) {
        for (int s = 0; s < A_STAGES; ++s) { mbar_init(bar_afull + 8 * s, 1); mbar_init(bar_aempty + 8 * s, 1); }
        for (int s = 0; s < B_STAGES; ++s) { mbar_init(bar_bfull + 8 * s, 1); mbar_init(bar_bempty + 8 * s, 1); }
        for (int a = 0; a < ACC; ++a) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 2 * DT_EPI_WARPS); }
        mbar_init(bar_bres, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), L::TMEM_COLS);
    tc_fence_before();
    cluster_sync_all();            // barriers of both CTAs initialised before any remote arrive or TMA completion
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();                    // everything above overlapped the previous kernel's last wave; tensors are touched from here on

    const long long tiles_img = (long long)p.tiles_x * p.tiles_y;
    const long long total_tiles = (long long)p.N * tiles_img;
    const long long ngroups = (total_tiles + 2 * MT - 1) / (2 * MT);     // a pair takes 2*MT consecutive tiles
    const long long total = ngroups * p.nblocks;
    const long long pair = blockIdx.x / 2, npairs = gridDim.x / 2;
    // with resident filters a pair keeps one filter block for the whole kernel
    const int my_nb = B_RESIDENT ? (int)(pair % p.nblocks) : 0;
    const long long first = B_RESIDENT ? (pair / p.nblocks) * p.nblocks + my_nb : pair;
    const long long step = B_RESIDENT ? (npairs / p.nblocks) * p.nblocks : npairs;

    // work item -> filter block and this CTA's mt-th tile (clamped to the last tile when the batch runs out: the
    // duplicate is computed and not stored)
    auto decode = [&](long long u, int mt, int& n, int& ty, int& tx, int& nb, bool& valid) {
        nb = (int)(u % p.nblocks);
        long long tl = (u / p.nblocks) * (2 * MT) + (long long)rank * MT + mt;
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
            const uint32_t filter_row0 = (uint32_t)(rank * (BN / 2));
            if (B_RESIDENT) {       // this CTA's half of all taps and chunks of the pair's filter block, once
                if (rank == 0 && issuer) mbar_arrive_expect_tx(bar_bres, (uint32_t)(2 * 9 * p.cchunks * L::B_TILE));
                const uint32_t bres_leader = mapa_shared(bar_bres, 0);
                for (int ch = 0; ch < p.cchunks; ++ch)
                    for (int tap = 0; tap < 9; ++tap)
                        if (issuer) tma_load_3d_pair(base + L::B_OFF + (ch * 9 + tap) * L::B_TILE, &tm_w, bres_leader, ch * CPC,
                                         my_nb * BN + filter_row0, tap);
            }
            unsigned long long acount = 0, bcount = 0;
            for (long long u = first; ok && u < total; u += step) {
                for (int ch = 0; ok && ch < p.cchunks; ++ch) {
                    int nb = 0;
                    for (int mt = 0; mt < MT; ++mt) {
                        int n, ty, tx; bool valid;
                        decode(u, mt, n, ty, tx, nb, valid);
                        const int st = (int)(acount % A_STAGES);
                        if (!mbar_wait_warp(bar_aempty + 8 * st, (uint32_t)(((acount / A_STAGES) & 1) ^ 1), abort_flag, p.status, DT_W_A_EMPTY)) { ok = false; break; }
                        if (rank == 0 && issuer) mbar_arrive_expect_tx(bar_afull + 8 * st, 2 * DT_A_BYTES);
                        if (issuer) tma_load_4d_pair(base + L::A_OFF + st * DT_A_STRIDE, &tm_x, mapa_shared(bar_afull + 8 * st, 0), ch * CPC,
                                         tx * DT_TW - p.pad, ty * DT_TH - p.pad, n);
                        ++acount;
                    }
                    if (!ok) break;
                    if (!B_RESIDENT) {
                        for (int tap = 0; tap < 9; ++tap) {
                            const int sb = (int)(bcount % B_STAGES);
                            if (!mbar_wait_warp(bar_bempty + 8 * sb, (uint32_t)(((bcount / B_STAGES) & 1) ^ 1), abort_flag, p.status, DT_W_B_EMPTY)) { ok = false; break; }
                            if (rank == 0 && issuer) mbar_arrive_expect_tx(bar_bfull + 8 * sb, 2 * L::B_TILE);
                            if (issuer) tma_load_3d_pair(base + L::B_OFF + sb * L::B_TILE, &tm_w, mapa_shared(bar_bfull + 8 * sb, 0), ch * CPC,
                                             nb * BN + filter_row0, tap);
                            ++bcount;
                        }
                    }
                }
            }
            if (!ok && issuer) drain_after_abort();
        }
    } else if (warp == 1) {
        // MMA issue (leader CTA only).  The whole warp runs the loop so that descriptors and addresses stay warp-uniform
        // values (issuing from a single-lane branch instead cost tens of cycles per tcgen05.mma, more than a 64-filter
        // MMA takes); one elected lane issues the tcgen05 instructions.
        if (rank == 0) {
            const bool issuer = elect_one();
            bool ok = true;
            if (B_RESIDENT) ok = mbar_wait_warp(bar_bres, 0, abort_flag, p.status, DT_W_B_RESIDENT);
            unsigned long long acount = 0, bcount = 0;
            int as = 0;
            uint32_t aphase = 0;
            for (long long u = first; ok && u < total; u += step) {
                if (!mbar_wait_warp(bar_tempty + 8 * as, aphase ^ 1, abort_flag, p.status, DT_W_T_EMPTY)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * MT * BN);
                for (int ch = 0; ok && ch < p.cchunks; ++ch) {
                    uint64_t a_desc0[MT];
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const int st = (int)((acount + mt) % A_STAGES);
                        if (!mbar_wait_warp(bar_afull + 8 * st, (uint32_t)(((acount + mt) / A_STAGES) & 1), abort_flag, p.status, DT_W_A_FULL)) { ok = false; break; }
                        a_desc0[mt] = smem_desc_k128_sbo(base + L::A_OFF + st * DT_A_STRIDE, DT_BOX_W * 128);
                    }
                    if (!ok) break;
                    tc_fence_after();
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
                        const uint64_t tap_shift = (uint64_t)((((tap / 3) * DT_BOX_W + (tap % 3)) * 128) >> 4);
#pragma unroll
                        for (int mt = 0; mt < MT; ++mt) {
                            const uint64_t a_desc = a_desc0[mt] + tap_shift;
#pragma unroll
                            for (int ks = 0; ks < 4; ++ks) {
                                if (tap == 0 && ks == 0)
                                    { if (issuer) tc_mma_pair<TF32>(d_tmem + mt * BN, a_desc, b_desc0, p.idesc, ch ? 1u : 0u); }
                                else
                                    { if (issuer) tc_mma_pair<TF32>(d_tmem + mt * BN, a_desc + (uint64_t)(ks * 2), b_desc0 + (uint64_t)(ks * 2), p.idesc, 1u); }
                            }
                        }
                        if (!B_RESIDENT) { if (issuer) tc_commit_pair(bar_bempty + 8 * sb, 3); ++bcount; }
                    }
                    if (!ok) break;
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) { if (issuer) tc_commit_pair(bar_aempty + 8 * (int)((acount + mt) % A_STAGES), 3); }
                    acount += MT;
                }
                if (ok && issuer) tc_commit_pair(bar_tfull + 8 * as, 3);
                if (++as == ACC) { as = 0; aphase ^= 1; }
            }
        }
    } else {
        const int quarter = warp % 4;
        const int half = (warp - 2) / 4;              // which half of the BN filter columns this warp drains
        const int l = quarter * 32 + lane;            // accumulator lane = pixel of the tile: h = l / 8, w = l % 8
        const int ph_ = l / DT_TW, pw_ = l % DT_TW;
        constexpr int CHUNKS = BN / 64;               // 32-column chunks per warp
        const uint32_t tempty_leader0 = mapa_shared(bar_tempty, 0);
        int as = 0;
        uint32_t aphase = 0;
        bool ok = true;
        [[maybe_unused]] bool stg_pending = false;
        // With one 32-filter chunk per warp the bias of that chunk stays in registers while the filter block does not
        // change (for resident filters: the whole kernel); eight 16-byte loads per accumulator tile otherwise.
        [[maybe_unused]] float4 bias_r[8];
        [[maybe_unused]] int bias_k0 = -1;
        for (long long u = first; ok && u < total; u += step) {
            if (!mbar_wait_bounded(bar_tfull + 8 * as, aphase, abort_flag, p.status, DT_W_T_FULL)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
                int n, ty, tx, nb; bool valid;
                decode(u, mt, n, ty, tx, nb, valid);
                const int oy = ty * DT_TH + ph_, ox = tx * DT_TW + pw_;
                const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((as * MT + mt) * BN + half * (BN / 2));
                bool writer;
                long long pix;
                if (p.pool) {
                    writer = valid && (oy >> 1) < p.PH && (ox >> 1) < p.PW;      // each lane of a window stores a quarter of its filters
                    pix = ((long long)n * p.PH + (oy >> 1)) * p.PW + (ox >> 1);
                } else {
                    writer = valid && oy < p.OH && ox < p.OW;
                    pix = ((long long)n * p.OH + oy) * p.OW + ox;
                }
#pragma unroll 1
                for (int chunk = 0; chunk < CHUNKS; ++chunk) {
                    uint32_t r[32];
                    tmem_ld_32x32(lane_addr + chunk * 32, r);
                    tmem_ld_wait();
                    if (mt == MT - 1 && chunk == CHUNKS - 1) {      // accumulator stage drained: release it on the leader
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * as);
                    }
                    const int k0 = nb * BN + half * (BN / 2) + chunk * 32;
                    auto load_bias4 = [&](int e) {
                        return (p.bias && k0 + e + 4 <= p.K) ? __ldg(reinterpret_cast<const float4*>(p.bias + k0 + e)) : make_float4(0.f, 0.f, 0.f, 0.f);
                    };
                    if constexpr (CHUNKS == 1) {
                        if (k0 != bias_k0) {
#pragma unroll
                            for (int e = 0; e < 32; e += 4) bias_r[e / 4] = load_bias4(e);
                            bias_k0 = k0;
                        }
                    }
                    auto bias4 = [&](int e) {
                        if constexpr (CHUNKS == 1) return bias_r[e / 4];
                        else return load_bias4(e);
                    };
                    if constexpr (TF32) {
                        // float storage: bias + ReLU, the 2x2 max with two shuffles per value, 16-byte stores
                        float v[32];
#pragma unroll
                        for (int e = 0; e < 32; e += 4) {
                            const float4 b4 = bias4(e);
                            v[e] = __uint_as_float(r[e]) + b4.x; v[e + 1] = __uint_as_float(r[e + 1]) + b4.y;
                            v[e + 2] = __uint_as_float(r[e + 2]) + b4.z; v[e + 3] = __uint_as_float(r[e + 3]) + b4.w;
                        }
                        if (p.relu) {
#pragma unroll
                            for (int e = 0; e < 32; ++e) v[e] = fmaxf(v[e], 0.f);
                        }
                        if (p.pool) {
                            uint32_t u[32];
#pragma unroll
                            for (int e = 0; e < 32; ++e) u[e] = __float_as_uint(v[e]);
                            pool2x2_split<32>(u, lane, [](uint32_t a, uint32_t b) { return __float_as_uint(fmaxf(__uint_as_float(a), __uint_as_float(b))); });
                            if (writer) {
                                const int f0 = pooled_first_word<32>(lane);          // this lane's 8 filters of the chunk
                                float* dst = reinterpret_cast<float*>(p.y) + pix * p.K + k0 + f0;
                                if (k0 + 32 <= p.K && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                                    reinterpret_cast<uint4*>(dst)[0] = make_uint4(u[0], u[1], u[2], u[3]);
                                    reinterpret_cast<uint4*>(dst)[1] = make_uint4(u[4], u[5], u[6], u[7]);
                                } else {
#pragma unroll
                                    for (int e = 0; e < 8; ++e)
                                        if (k0 + f0 + e < p.K) dst[e] = __uint_as_float(u[e]);
                                }
                            }
                        } else if (writer) {
                            float* dst = reinterpret_cast<float*>(p.y) + pix * p.K + k0;
                            if (k0 + 32 <= p.K && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                                for (int c = 0; c < 8; ++c) reinterpret_cast<float4*>(dst)[c] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
                            } else {
#pragma unroll
                                for (int e = 0; e < 32; ++e)
                                    if (k0 + e < p.K) dst[e] = v[e];
                            }
                        }
                    } else {
                    // bias + ReLU, packed to bf16 pairs; the 2x2 max is taken on the packed values (rounding is monotonic)
                    uint32_t w[16];
#pragma unroll
                    for (int e = 0; e < 32; e += 4) {
                        const float4 b4 = bias4(e);
                        float v0 = __uint_as_float(r[e]) + b4.x, v1 = __uint_as_float(r[e + 1]) + b4.y;
                        float v2 = __uint_as_float(r[e + 2]) + b4.z, v3 = __uint_as_float(r[e + 3]) + b4.w;
                        if (p.relu) { v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f); v2 = fmaxf(v2, 0.f); v3 = fmaxf(v3, 0.f); }
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(v0, v1), h1 = __floats2bfloat162_rn(v2, v3);
                        w[e / 2] = *reinterpret_cast<uint32_t*>(&h0);
                        w[e / 2 + 1] = *reinterpret_cast<uint32_t*>(&h1);
                    }
                    if (p.pool) {
                        pool2x2_split<16>(w, lane, [](uint32_t a, uint32_t b) {
                            const __nv_bfloat162 m = __hmax2(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
                            return *reinterpret_cast<const uint32_t*>(&m);
                        });
                        if (writer) {
                            const int f0 = 2 * pooled_first_word<16>(lane);          // this lane's 8 filters of the chunk
                            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.y) + pix * p.K + k0 + f0;
                            if (k0 + 32 <= p.K && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                                *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                            } else {
#pragma unroll
                                for (int e = 0; e < 8; ++e)
                                    if (k0 + f0 + e < p.K) dst[e] = reinterpret_cast<const __nv_bfloat16*>(w)[e];
                            }
                        }
                    } else if (STG) {
                        // Unpooled outputs leave through the TMA unit: the warp lays its 32 pixels x 64 filters out as a
                        // 128-byte-swizzled box (8 wide, 4 high) in its own staging tile and one lane stores it; the
                        // box is clipped at the image and filter edges.  Stored from registers instead, every 16-byte
                        // store instruction of a warp touches 32 different lines.
                        uint8_t* stg = gen + L::STG_OFF + (warp - 2) * 4096;
                        if (chunk == 0 && stg_pending) {       // the previous store must have read the tile
                            if (lane == 0) tma_store_wait_read<0>();
                            __syncwarp();
                            stg_pending = false;
                        }
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            *reinterpret_cast<uint4*>(stg + lane * 128 + (((chunk * 4 + c) ^ (lane & 7)) << 4)) =
                                make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
                        if (chunk == CHUNKS - 1) {
                            fence_async_shared();
                            __syncwarp();
                            if (lane == 0 && valid) {
                                tma_store_4d(&tm_y, base + L::STG_OFF + (warp - 2) * 4096, nb * BN + half * (BN / 2), tx * DT_TW,
                                             ty * DT_TH + 4 * quarter, n);
                                tma_store_commit();
                            }
                            stg_pending = true;
                        }
                    } else if (writer) {
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
                }
            }
            if (++as == ACC) { as = 0; aphase ^= 1; }
        }
        if (STG && lane == 0) tma_store_wait_all();      // staged outputs are on their way before the CTA leaves
    }

    // neither CTA may leave (or give back tensor memory) while its partner can still read its shared memory,
    // signal its barriers or run an MMA over both tensor memories
    tc_fence_before();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, L::TMEM_COLS);
    }
}

template <int BN, int MT, int A_STAGES, int B_STAGES, bool B_RESIDENT, int RES_CHUNKS, bool TF32, bool STG = false>
int run2(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const DtParams& p, cudaStream_t st, const CUtensorMap* tm_y = nullptr) {
    using L = Dt2Smem<BN, MT, A_STAGES, B_STAGES, B_RESIDENT, RES_CHUNKS, STG>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA exceeded");
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(direct_tc2_kernel<BN, MT, A_STAGES, B_STAGES, B_RESIDENT, RES_CHUNKS, TF32, STG>,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    WINO_CUDA_CHECK(attr_err);
    const long long total_tiles = (long long)p.N * p.tiles_x * p.tiles_y;
    const long long total = (total_tiles + 2 * MT - 1) / (2 * MT) * p.nblocks;
    long long pairs = sm_count() / 2;
    if (total < pairs) pairs = total;
    if (B_RESIDENT) pairs = pairs / p.nblocks * p.nblocks;      // every pair owns one filter block
    if (pairs < 1) pairs = p.nblocks;
    ProfScope prof(STAGE_DIRECT_TC, st);
    count_launch();
    WINO_CUDA_CHECK(launch_kernel(direct_tc2_kernel<BN, MT, A_STAGES, B_STAGES, B_RESIDENT, RES_CHUNKS, TF32, STG>, dim3((unsigned)(2 * pairs)),
                                  dim3(DT_THREADS), L::TOTAL, st, pdl_enabled(), tm_x, tm_w, tm_y ? *tm_y : tm_x, p));
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

// 0: never, 1 (default): where it is the faster kernel, 2: wherever it can run
int pair_mode() {
    static const int mode = [] { const char* e = getenv("WINO_DIRECT_TC_PAIR"); return e ? atoi(e) : 1; }();
    return mode;
}
// experiment knob: "<bn>,<mt>,<resident>" overrides the variant choice
bool variant_override(int& bn, int& mt, int& resident) {
    const char* e = getenv("WINO_DIRECT_TC_VARIANT");
    return e && sscanf(e, "%d,%d,%d", &bn, &mt, &resident) == 3;
}

}  // namespace

bool direct_tc2_applies(const wino_conv_desc& d) {
    if (pair_mode() == 0) return false;
    if (!(d.layout_in == WINO_NHWC && d.layout_out == WINO_NHWC && d.k % 16 == 0 && d.k >= 64)) return false;
    return d.dtype == WINO_BF16 ? d.c % 64 == 0 : d.dtype == WINO_TF32 ? d.c % 32 == 0 : false;
}

bool direct_tc_stores_nchw(const wino_conv_desc& d) {
    int obn, omt, ores;
    return direct_tc2_applies(d) && direct_tc2t_applies(d) && !variant_override(obn, omt, ores);
}

int launch_direct_tc2(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                      cudaStream_t st, bool y_nchw) {
    if (d.n == 0) return WINO_OK;
    if (direct_tc_stores_nchw(d)) return launch_direct_tc2t(d, g, x, packed, bias, y, st, y_nchw);
    if (y_nchw) return fail(WINO_E_UNSUPPORTED, "direct conv (CTA pairs): this kernel variant stores NHWC only");
    if (((uintptr_t)x | (uintptr_t)packed | (uintptr_t)y | (d.has_bias ? (uintptr_t)bias : 0)) & 15)
        return fail(WINO_E_BADARG, "direct conv: buffers (and the bias) must be 16-byte aligned");
    DtParams p;
    p.bias = d.has_bias ? bias : nullptr; p.y = y;
    p.N = d.n; p.OH = g.oh; p.OW = g.ow; p.K = d.k; p.pad = d.pad; p.PH = g.ph; p.PW = g.pw;
    p.tiles_x = (g.ow + DT_TW - 1) / DT_TW; p.tiles_y = (g.oh + DT_TH - 1) / DT_TH;
    const bool tf32 = d.dtype == WINO_TF32;
    const int es = tf32 ? 4 : 2;
    p.cchunks = d.c / (128 / es);
    p.relu = d.relu; p.pool = d.pool2x2; p.y_nchw = 0;
    int rc = status_word(&p.status);
    if (rc) return rc;
    int bn = d.k >= 256 ? 256 : d.k >= 128 ? 128 : 64, mt = 1, resident = 0;
    if (p.cchunks == 1 && bn <= 128) resident = 1;
    else if (p.cchunks == 2 && bn <= 128) resident = 1;
    if (bn == 128 && !resident) mt = 2;
    if (bn == 64) mt = 2;
    variant_override(bn, mt, resident);
    p.nblocks = (d.k + bn - 1) / bn;
    p.idesc = make_idesc(tf32 ? OP_TF32 : OP_BF16, bn, 256);
    CUtensorMap tm_x, tm_w;
    {
        const unsigned long long dims[4] = {(unsigned long long)d.c, (unsigned long long)d.w, (unsigned long long)d.h, (unsigned long long)d.n};
        const unsigned long long ues = (unsigned long long)es;
        const unsigned long long strides[3] = {d.c * ues, (unsigned long long)d.w * d.c * ues, (unsigned long long)d.h * d.w * d.c * ues};
        const unsigned box[4] = {(unsigned)(128 / es), (unsigned)DT_BOX_W, (unsigned)DT_BOX_H, 1u};
        if ((rc = encode_tensor_map(&tm_x, tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x, dims, strides, box, true))) return rc;
    }
    // each CTA of a pair loads half of the filter block's rows per tap
    if ((rc = make_map_k128(&tm_w, tf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, es, packed, d.c, d.k, d.k, 9, bn / 2))) return rc;
    const int key = bn * 100 + mt * 10 + resident * (p.cchunks <= 2 ? p.cchunks : 9);
    static const bool stage_off = [] { const char* e = getenv("WINO_DIRECT_TC_TMA_STORE"); return e && e[0] == '0'; }();
    if (!stage_off && !tf32 && !d.pool2x2 && key == 128 * 100 + 11 && d.k % 8 == 0) {
        // unpooled bf16 output of a resident 64-channel layer (64 -> 128 of VGG-16): stores staged through the TMA unit
        CUtensorMap tm_y;
        const unsigned long long dims[4] = {(unsigned long long)d.k, (unsigned long long)g.ow, (unsigned long long)g.oh, (unsigned long long)d.n};
        const unsigned long long strides[3] = {d.k * 2ull, (unsigned long long)g.ow * d.k * 2ull, (unsigned long long)g.oh * g.ow * d.k * 2ull};
        const unsigned box[4] = {64u, (unsigned)DT_TW, 4u, 1u};
        if ((rc = encode_tensor_map(&tm_y, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, y, dims, strides, box, true))) return rc;
        return run2<128, 1, 4, 2, true, 1, false, true>(tm_x, tm_w, p, st, &tm_y);
    }
    switch (key) {
        case 64 * 100 + 11:  return tf32 ? run2<64, 1, 6, 2, true, 1, true>(tm_x, tm_w, p, st) : run2<64, 1, 6, 2, true, 1, false>(tm_x, tm_w, p, st);
        case 64 * 100 + 21:  return tf32 ? run2<64, 2, 6, 2, true, 1, true>(tm_x, tm_w, p, st) : run2<64, 2, 6, 2, true, 1, false>(tm_x, tm_w, p, st);
        case 64 * 100 + 41:  return tf32 ? run2<64, 4, 8, 2, true, 1, true>(tm_x, tm_w, p, st) : run2<64, 4, 8, 2, true, 1, false>(tm_x, tm_w, p, st);
        case 128 * 100 + 11: return tf32 ? run2<128, 1, 6, 2, true, 1, true>(tm_x, tm_w, p, st) : run2<128, 1, 6, 2, true, 1, false>(tm_x, tm_w, p, st);
        case 128 * 100 + 21: return tf32 ? run2<128, 2, 6, 2, true, 1, true>(tm_x, tm_w, p, st) : run2<128, 2, 6, 2, true, 1, false>(tm_x, tm_w, p, st);
        case 128 * 100 + 12: return tf32 ? run2<128, 1, 3, 2, true, 2, true>(tm_x, tm_w, p, st) : run2<128, 1, 3, 2, true, 2, false>(tm_x, tm_w, p, st);
        case 64 * 100 + 22:  return tf32 ? run2<64, 2, 6, 2, true, 2, true>(tm_x, tm_w, p, st) : run2<64, 2, 6, 2, true, 2, false>(tm_x, tm_w, p, st);
        case 64 * 100 + 20:  return tf32 ? run2<64, 2, 6, 9, false, 1, true>(tm_x, tm_w, p, st) : run2<64, 2, 6, 9, false, 1, false>(tm_x, tm_w, p, st);
        case 128 * 100 + 10: return tf32 ? run2<128, 1, 6, 6, false, 1, true>(tm_x, tm_w, p, st) : run2<128, 1, 6, 6, false, 1, false>(tm_x, tm_w, p, st);
        case 128 * 100 + 20: return tf32 ? run2<128, 2, 6, 6, false, 1, true>(tm_x, tm_w, p, st) : run2<128, 2, 6, 6, false, 1, false>(tm_x, tm_w, p, st);
        case 256 * 100 + 10: return tf32 ? run2<256, 1, 4, 6, false, 1, true>(tm_x, tm_w, p, st) : run2<256, 1, 4, 6, false, 1, false>(tm_x, tm_w, p, st);
        default: return fail(WINO_E_UNSUPPORTED, "direct conv (CTA pairs): no kernel variant for this shape");
    }
}

}  // namespace wino

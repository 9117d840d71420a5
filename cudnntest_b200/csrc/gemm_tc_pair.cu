// Tensor-core batched tile GEMM on CTA pairs (sm_100a):  M[xi][t][k] = sum_c V[xi][t][c] * U[xi][k][c]
// for wide layers (at least 256 filters, long contractions).
//
// Same role as gemm_tc.cu (GEMM_batch_256_128x128_KMKN / _MKNK of the reference, comparison/GEMM.cuh:124-255, :4-122),
// different tile: a single CTA multiplying 128 tiles x 256 filters has to pull 48 KB of operands out of the L2 for
// every 64-deep slice of the contraction, which at 512 channels is more than the L2 delivers (the single-CTA kernel
// runs its tensor pipe 45 % of the time on the 512 -> 512 layers).  Here two CTAs of a cluster form one
// tcgen05.mma.cta_group::2 tile of 256 tiles x 256 filters: each CTA loads its own 128 tile rows of V and only HALF of the
// 256 filter rows of U (the MMA unit reads the other half from the partner's shared memory), i.e. 32 KB per slice for
// the same arithmetic, two thirds of the L2 traffic.  No TMA multicast is used.
//
//   * work unit = (xi, pair of 128-tile row blocks, 256-filter column block), column block fastest so that the pairs
//     working side by side share the same V rows through the L2;
//   * warp 0 of each CTA: TMA producer for its own V rows and its half of the U rows (cp.async.bulk.tensor.3d ...
//     cta_group::2, completion bytes counted on the LEADER's "full" mbarrier);
//   * warp 1 of the leader: one elected lane issues tcgen05.mma.cta_group::2 (M = 256, N = 256, 32 bytes of K per
//     instruction) into one of two 256-column accumulators that span both CTAs' tensor memory; its commits arrive on
//     the ring-slot and accumulator barriers of BOTH CTAs (tcgen05.commit ... multicast::cluster, an mbarrier signal);
//   * warps 2-5 of each CTA: epilogue of that CTA's 128 accumulator lanes, as in gemm_tc.cu: tcgen05.ld 32 columns,
//     128-byte-swizzled 32 x 32 float staging tile, TMA store (rows past the tile count and columns past Kq clipped).
//     With M24 the products leave in 3 bytes each: 64 columns at a time, rounded to their upper 24 bits, as a
//     128-byte-swizzled 64 x 32 tile of 16-bit upper halves and a 64-byte-swizzled tile of third bytes, two TMA stores
//     into two planes of the product buffer (output_transform.cu reads them back).
// Every mbarrier wait is bounded; a wait that gives up raises its CTA's abort flag, records a code, and both CTAs meet
// at the final cluster barrier (the partner's waits run out too) before tensor memory is released.
// Bound: the product write (a*a*T*Kq*4 bytes, 3 with M24) against 2*a*a*T*C*K flops, and the operand fill: at 512
// channels the pair pulls 2 x 256 KB out of the L2 per work unit, 7 TB/s over the chip at the measured speed.
#include <cstdlib>
#include <mutex>

#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace wino {

namespace {

constexpr int TP_THREADS = 192;
constexpr int TP_BN = 256;                       // filters per pair tile
constexpr int TP_B_BYTES = (TP_BN / 2) * TC_ROW_BYTES;   // each CTA holds half of the filter rows of a ring slot
constexpr int TP_STORE_TILE = 32 * 32 * 4;       // one epilogue staging tile: 32 rows x 32 floats
constexpr int TP_EPI_WARPS = 4;

enum TpWaitCode { TP_WAIT_EMPTY = 21, TP_WAIT_FULL = 22, TP_WAIT_TMEM_EMPTY = 23, TP_WAIT_TMEM_FULL = 24 };

struct TpParams {
    long long t_rows;
    int kq, cp;
    int batches, mpairs, nblocks, kchunks;
    uint32_t idesc;
    int* status;
};

constexpr int TP_STORE_TILE24 = 32 * 128 + 32 * 64;   // 3-byte products: 32 rows x 64 upper halves + 32 rows x 64 third bytes

template <int STAGES, bool M24 = false>
struct TpSmem {
    static constexpr int A_OFF = 0;
    static constexpr int B_OFF = STAGES * TC_A_BYTES;
    static constexpr int STORE_OFF = B_OFF + STAGES * TP_B_BYTES;          // 4 warps x 2 staging tiles of 4 (6) KiB
    static constexpr int STORE_TILE = M24 ? TP_STORE_TILE24 : TP_STORE_TILE;
    static constexpr int BAR_OFF = STORE_OFF + 2 * TP_EPI_WARPS * STORE_TILE;   // full[STAGES], empty[STAGES], tfull[2], tempty[2]
    static constexpr int SLOT_OFF = BAR_OFF + 8 * (2 * STAGES + 4);
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;
};

// M24: the products leave as the upper 24 bits of each float (rounded to nearest), split into a plane of 16-bit upper
// halves (tm_m) and a plane of third bytes (tm_lo): 3 bytes per product through HBM instead of 4, and again when the
// output transform reads them.
template <bool TF32, int STAGES, bool M24>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(TP_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_u,
                    const __grid_constant__ CUtensorMap tm_m, const __grid_constant__ CUtensorMap tm_lo, const TpParams p) {
    using L = TpSmem<STAGES, M24>;
    constexpr int ESIZE = TF32 ? 4 : 2;
    constexpr int KC = TC_ROW_BYTES / ESIZE;        // contraction elements per ring slot
    constexpr int UMMA_K = 32 / ESIZE;              // contraction elements per tcgen05.mma

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;       // same offset in both CTAs of the pair
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_ring = base + L::A_OFF, b_ring = base + L::B_OFF;
    const uint32_t bar_full = base + L::BAR_OFF, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::SLOT_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::SLOT_OFF + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t rank = cluster_ctarank();          // 0 = leader (issues the MMAs, owns the "full" and "tempty" barriers)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 2 * TP_EPI_WARPS);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(smem_u32((const void*)tmem_slot), 512);
    tc_fence_before();
    cluster_sync_all();            // barriers of both CTAs initialised before any remote arrive or TMA completion
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long total = (long long)p.batches * p.mpairs * p.nblocks;
    const long long pair = blockIdx.x / 2, npairs = gridDim.x / 2;

    auto decode = [&](long long u, int& xi, int& mp, int& nb) {
        nb = (int)(u % p.nblocks);
        mp = (int)((u / p.nblocks) % p.mpairs);
        xi = (int)(u / ((long long)p.nblocks * p.mpairs));
    };

    if (warp == 0) {
        {   // the whole warp walks the ring (warp-uniform addresses); one elected lane issues the copies
            const bool issuer = elect_one();
            const uint32_t full_leader = mapa_shared(bar_full, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long u = pair; ok && u < total; u += npairs) {
                int xi, mp, nb;
                decode(u, xi, mp, nb);
                const int row0 = (mp * 2 + (int)rank) * TC_BM;                  // this CTA's 128 tile rows
                const int frow0 = nb * TP_BN + (int)rank * (TP_BN / 2);          // this CTA's half of the filter rows
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, TP_WAIT_EMPTY)) { ok = false; break; }
                    if (rank == 0 && issuer) mbar_arrive_expect_tx(bar_full + 8 * stage, 2 * (TC_A_BYTES + TP_B_BYTES));
                    if (issuer) {
                        tma_load_3d_pair(a_ring + stage * TC_A_BYTES, &tm_v, full_leader + 8 * stage, kc * KC, row0, xi);
                        tma_load_3d_pair(b_ring + stage * TP_B_BYTES, &tm_u, full_leader + 8 * stage, kc * KC, frow0, xi);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok && issuer) drain_after_abort();
        }
    } else if (warp == 1) {
        if (rank == 0) {   // warp-uniform loop, one elected lane issues the tcgen05 instructions
            const bool issuer = elect_one();
            int stage = 0, as = 0;
            uint32_t phase = 0, aphase = 0;
            bool ok = true;
            for (long long u = pair; ok && u < total; u += npairs) {
                if (!mbar_wait_warp(bar_tempty + 8 * as, aphase ^ 1, abort_flag, p.status, TP_WAIT_TMEM_EMPTY)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * TP_BN);
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    if (!mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, p.status, TP_WAIT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const int left = p.cp - kc * KC;
                    const int ksteps = left >= KC ? KC / UMMA_K : (left + UMMA_K - 1) / UMMA_K;
                    // descriptors once per ring slot (CTA-relative: the same offsets in both CTAs); a K-step adds 32 bytes
                    const uint64_t a_desc = smem_desc_k128(a_ring + stage * TC_A_BYTES), b_desc = smem_desc_k128(b_ring + stage * TP_B_BYTES);
#pragma unroll 4
                    for (int ks = 0; ks < ksteps; ++ks)
                        if (issuer) tc_mma_pair<TF32>(d_tmem, a_desc + (uint64_t)(ks * 2), b_desc + (uint64_t)(ks * 2), p.idesc, (kc | ks) ? 1u : 0u);
                    if (issuer) tc_commit_pair(bar_empty + 8 * stage, 3);       // frees the slot in both CTAs
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok && issuer) tc_commit_pair(bar_tfull + 8 * as, 3);        // accumulator ready in both CTAs
                as ^= 1;
                if (as == 0) aphase ^= 1;
            }
        }
    } else {
        const int quarter = warp % 4;                 // tensor-memory lanes [32*quarter, 32*quarter + 32)
        uint8_t* stage_gen = gen_base + L::STORE_OFF + quarter * 2 * L::STORE_TILE;
        const uint32_t stage_s = base + L::STORE_OFF + quarter * 2 * L::STORE_TILE;
        const uint32_t tempty_leader = mapa_shared(bar_tempty, 0);
        int as = 0;
        uint32_t aphase = 0, issued = 0;
        bool ok = true;
        for (long long u = pair; ok && u < total; u += npairs) {
            int xi, mp, nb;
            decode(u, xi, mp, nb);
            if (!mbar_wait_bounded(bar_tfull + 8 * as, aphase, abort_flag, p.status, TP_WAIT_TMEM_FULL)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const long long row0 = (long long)(mp * 2 + (int)rank) * TC_BM + quarter * 32;
            if constexpr (M24) {
#pragma unroll 1
                for (int unit = 0; unit < TP_BN / 64; ++unit) {       // 64 columns at a time
                    uint32_t r[64];
                    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * TP_BN + unit * 64);
                    tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
                    tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
                    tmem_ld_wait();
                    if (unit == TP_BN / 64 - 1) {     // this warp's share of the accumulator is in registers
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * as);
                    }
                    const int col0 = nb * TP_BN + unit * 64;
                    if (row0 < p.t_rows && col0 < p.kq) {
                        const uint32_t buf = issued & 1;
                        if (issued >= 2) {            // the stores that last used this staging tile must have read it
                            if (lane == 0) tma_store_wait_read<1>();
                            __syncwarp();
                        }
#pragma unroll
                        for (int i = 0; i < 64; ++i) r[i] += 0x80u;       // round the 24 kept bits to nearest
                        // upper halves: 64 x 2 bytes per row, 128-byte swizzle (16-byte chunk index XOR row mod 8)
                        uint4* hi = reinterpret_cast<uint4*>(stage_gen + buf * L::STORE_TILE + lane * 128);
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            hi[j ^ (lane & 7)] = make_uint4(__byte_perm(r[8 * j], r[8 * j + 1], 0x7632), __byte_perm(r[8 * j + 2], r[8 * j + 3], 0x7632),
                                                            __byte_perm(r[8 * j + 4], r[8 * j + 5], 0x7632), __byte_perm(r[8 * j + 6], r[8 * j + 7], 0x7632));
                        // third bytes: 64 bytes per row, 64-byte swizzle (chunk index XOR (row / 2) mod 4)
                        uint4* lo = reinterpret_cast<uint4*>(stage_gen + buf * L::STORE_TILE + 32 * 128 + lane * 64);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t w[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const uint32_t* q = &r[16 * j + 4 * e];
                                w[e] = __byte_perm(__byte_perm(q[0], q[1], 0x0051), __byte_perm(q[2], q[3], 0x0051), 0x5410);
                            }
                            lo[j ^ ((lane >> 1) & 3)] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                        fence_async_shared();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(&tm_m, stage_s + buf * L::STORE_TILE, col0, (int)row0, xi);
                            tma_store_3d(&tm_lo, stage_s + buf * L::STORE_TILE + 32 * 128, col0, (int)row0, xi);
                            tma_store_commit();
                        }
                        ++issued;
                    }
                }
            } else {
#pragma unroll 1
            for (int chunk = 0; chunk < TP_BN / 32; ++chunk) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * TP_BN + chunk * 32), r);
                tmem_ld_wait();
                if (chunk == TP_BN / 32 - 1) {        // this warp's share of the accumulator is in registers
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(tempty_leader + 8 * as);
                }
                const int col0 = nb * TP_BN + chunk * 32;
                if (row0 < p.t_rows && col0 < p.kq) {
                    const uint32_t buf = issued & 1;
                    if (issued >= 2) {                // the store that last used this staging tile must have read it
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                    }
                    float4* dst = reinterpret_cast<float4*>(stage_gen + buf * TP_STORE_TILE + lane * 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        dst[j ^ (lane & 7)] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    fence_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&tm_m, stage_s + buf * TP_STORE_TILE, col0, (int)row0, xi);
                        tma_store_commit();
                    }
                    ++issued;
                }
            }
            }
            as ^= 1;
            if (as == 0) aphase ^= 1;
        }
        if (lane == 0) tma_store_wait_all();
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

template <bool TF32, int STAGES, bool M24>
int run(const CUtensorMap& tm_v, const CUtensorMap& tm_u, const CUtensorMap& tm_m, const CUtensorMap& tm_lo, const TpParams& p,
        cudaStream_t st) {
    using L = TpSmem<STAGES, M24>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA exceeded");
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(gemm_tc_pair_kernel<TF32, STAGES, M24>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    WINO_CUDA_CHECK(attr_err);
    const long long total = (long long)p.batches * p.mpairs * p.nblocks;
    long long pairs = sm_count() / 2;
    if (total < pairs) pairs = total;
    if (pairs < 1) pairs = 1;
    ProfScope prof(STAGE_GEMM, st);
    count_launch();
    gemm_tc_pair_kernel<TF32, STAGES, M24><<<(unsigned)(2 * pairs), TP_THREADS, L::TOTAL, st>>>(tm_v, tm_u, tm_m, tm_lo, p);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace

// 0: never, 1 (default): layers with at least 256 filters and 512 channels, 2: every layer with at least 256 filters
static int gemm_pair_mode() {
    static const int mode = [] { const char* e = getenv("WINO_GEMM_PAIR"); return e ? atoi(e) : 1; }();
    return mode;
}

bool gemm_tc_pair_applies(int k, int cp, long long t_rows) {
    const int mode = gemm_pair_mode();
    if (mode == 0 || k < 256 || t_rows < 2 * TC_BM) return false;
    return mode >= 2 || cp >= 512;
}

// 3-byte products: for layers the pair kernel takes, filters padded to a multiple of 16 (the row pitch of the byte plane)
bool gemm_tc_m24_applies(int operand, int k, int cp, int kq, long long t_rows) {
    static const bool off = [] { const char* e = getenv("WINO_M24"); return e && e[0] == '0'; }();
    static const bool bn_forced = [] { const char* e = getenv("WINO_GEMM_BN"); return e && atoi(e) > 0; }();
    return !off && !bn_forced && (operand == OP_TF32 || operand == OP_BF16 || operand == OP_F16) && kq % 16 == 0 &&
           gemm_tc_pair_applies(k, cp, t_rows);
}

int launch_gemm_tc_pair(int operand, const void* v, const void* u, float* m, int batches, long long t_rows, long long tp,
                        int k, int cp, int kq, cudaStream_t st, bool m24) {
    if (t_rows <= 0) return WINO_OK;
    if (operand != OP_TF32 && operand != OP_BF16 && operand != OP_F16)
        return fail(WINO_E_BADARG, "gemm_tc_pair: bad operand kind %d", operand);
    const int es = operand == OP_TF32 ? 4 : 2;
    if ((cp * es) % 16 != 0 || kq % 4 != 0) return fail(WINO_E_BADARG, "gemm_tc_pair: row pitch must be a multiple of 16 bytes");
    if (((uintptr_t)v | (uintptr_t)u | (uintptr_t)m) & 15) return fail(WINO_E_BADARG, "gemm_tc_pair: buffers must be 16-byte aligned");
    const CUtensorMapDataType dt = operand_map_type(operand);
    CUtensorMap tm_v, tm_u, tm_m;
    int rc;
    if ((rc = make_map_k128(&tm_v, dt, es, v, cp, t_rows, tp, batches, TC_BM))) return rc;
    if ((rc = make_map_k128(&tm_u, dt, es, u, cp, k, k, batches, TP_BN / 2))) return rc;
    CUtensorMap tm_lo;
    if (m24) {
        if (kq % 16 != 0) return fail(WINO_E_BADARG, "gemm_tc_pair: 3-byte products need a filter pitch that is a multiple of 16");
        // plane of upper halves: [batches][tp][kq] 16-bit, boxes of 64 x 32; plane of third bytes behind it, 64-byte swizzle
        if ((rc = make_map_k128(&tm_m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, m, kq, t_rows, tp, batches, 32))) return rc;
        const unsigned long long dims[3] = {(unsigned long long)kq, (unsigned long long)t_rows, (unsigned long long)batches};
        const unsigned long long strides[2] = {(unsigned long long)kq, (unsigned long long)tp * kq};
        const unsigned box[3] = {64u, 32u, 1u};
        const char* lo_plane = reinterpret_cast<const char*>(m) + (long long)batches * tp * kq * 2;
        if ((rc = encode_tensor_map(&tm_lo, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, lo_plane, dims, strides, box, 2))) return rc;
    } else {
        if ((rc = make_map_k128(&tm_m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, m, kq, t_rows, tp, batches, 32))) return rc;
        tm_lo = tm_m;
    }
    TpParams p;
    p.t_rows = t_rows; p.cp = cp; p.kq = kq; p.batches = batches;
    const long long mblocks = (t_rows + TC_BM - 1) / TC_BM;
    p.mpairs = (int)((mblocks + 1) / 2);
    p.nblocks = (k + TP_BN - 1) / TP_BN;
    p.kchunks = (cp * es + TC_ROW_BYTES - 1) / TC_ROW_BYTES;
    p.idesc = make_idesc(operand, TP_BN, 2 * TC_BM);
    if ((rc = status_word(&p.status))) return rc;
    if (m24) return operand == OP_TF32 ? run<true, 5, true>(tm_v, tm_u, tm_m, tm_lo, p, st) : run<false, 5, true>(tm_v, tm_u, tm_m, tm_lo, p, st);
    return operand == OP_TF32 ? run<true, 5, false>(tm_v, tm_u, tm_m, tm_lo, p, st) : run<false, 5, false>(tm_v, tm_u, tm_m, tm_lo, p, st);
}

}  // namespace wino

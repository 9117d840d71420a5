// Split-TF32 batched tile GEMM for sm_100a (the FP32X3 variant):  M[xi][t][k] = sum_c V[xi][t][c] * U[xi][k][c]
// with FP32 operands and FP32-level accuracy on the TF32 tensor-core path.
//
// Takes the role of GEMM_batch_256_128x128_KMKN / _MKNK (comparison/GEMM.cuh:124-255, :4-122), whose arithmetic is
// FP32 FFMA.  Every operand value x is used as a TF32 head and a TF32 tail, x = hi + lo with hi = tf32(x) and
// lo = tf32(x - hi), and each product is rebuilt from three TF32 products, lo(V)*hi(U) + hi(V)*lo(U) + hi(V)*hi(U),
// accumulated in FP32 in tensor memory.  The two cross terms go to an accumulator of their own and are added to the head*head
// accumulator in the epilogue: the tensor core truncates when it adds into an accumulator, and cross terms added one
// ring slot at a time to an already large sum would lose their low bits on every addition.  Measured on a 512-deep
// contraction: max|y - oracle| / max|oracle| = 6e-6, against 1.7e-5 for the FFMA tile GEMM.  The dropped lo*lo term
// is below 2^-22 of the product.
//
// V arrives as plain FP32 rows of Cp floats, exactly what the input transform of the FP32 variant writes: it is split
// INSIDE the kernel, so the largest buffer of the pipeline crosses HBM once in each direction at 4 bytes per value
// instead of 8.  U (small, written once per weight tensor) arrives pre-split: rows of 2*Cp floats, heads then tails.
//
//   * warp 0: TMA producer.  Per ring slot one 128-row x 128-byte box of V and two BN-row boxes of U (heads, tails);
//   * warps 6-9: converters.  When a slot's bytes have landed, each thread takes eight 16-byte units of the V tile,
//     overwrites them with the heads and writes the tails at the same offsets of a second tile (the split is
//     element-wise, so the 128-byte swizzle the TMA unit applied carries over), then makes the writes visible to
//     the tensor-core proxy (fence.proxy.async) and arrives on the slot's "converted" barrier;
//   * warp 1: one elected lane issues three groups of tcgen05.mma (kind::tf32, M = 128, N = BN, 8 floats of K each)
//     per slot and commits the slot back to the producer;
//   * warps 2-5: epilogue as in gemm_tc.cu (tcgen05.ld, swizzled staging, TMA stores of FP32 M).
// No TMA multicast, no clusters.  Every mbarrier wait is bounded; a wait that gives up records its code, raises the
// CTA's abort flag, and the CTA frees its tensor memory and returns.
#include <mutex>

#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace wino {

namespace {

constexpr int TS_THREADS = 320;
constexpr int TS_STORE_TILE = 32 * 32 * 4;
constexpr int TS_KC = TC_ROW_BYTES / 4;   // floats of contraction per ring slot
constexpr int TS_UMMA_K = 8;              // floats of contraction per tcgen05.mma (32 bytes)

enum TsWaitCode { TS_WAIT_EMPTY = 21, TS_WAIT_FULL = 22, TS_WAIT_TMEM_EMPTY = 23, TS_WAIT_TMEM_FULL = 24, TS_WAIT_CONVERTED = 25 };

struct TsParams {
    long long t_rows;
    int kq, cp;
    int batches, mblocks, nblocks, kchunks;
    uint32_t idesc;
    int* status;
};

template <int BN, int STAGES>
struct TsSmem {
    static constexpr int B_BYTES = BN * TC_ROW_BYTES;
    static constexpr int SLOT = 2 * TC_A_BYTES + 2 * B_BYTES;        // V heads (in place), V tails, U heads, U tails
    static constexpr int RING = STAGES * SLOT;
    static constexpr int STORE_OFF = RING;                           // 4 warps x 2 staging tiles of 4 KiB
    static constexpr int BAR_OFF = STORE_OFF + 8 * TS_STORE_TILE;    // full, converted, empty [STAGES]; tfull[2], tempty[2]
    static constexpr int SLOT_OFF = BAR_OFF + 8 * (3 * STAGES + 4);
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;               // + slack for the 1 KiB alignment of the ring
};

template <int BN, int STAGES>
__global__ void __launch_bounds__(TS_THREADS, 1)
gemm_tc_split_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_u,
                     const __grid_constant__ CUtensorMap tm_m, const TsParams p) {
    using L = TsSmem<BN, STAGES>;
    constexpr uint32_t TMEM_COLS = 4 * BN;   // two stages x (head*head accumulator, cross-term accumulator): 256 or 512 columns

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bar_full = base + L::BAR_OFF, bar_conv = bar_full + 8 * STAGES, bar_empty = bar_conv + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::SLOT_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::SLOT_OFF + 4);
    // slot s: [V heads | V tails | U heads | U tails]
    auto v_hi = [&](int s) { return base + (uint32_t)(s * L::SLOT); };
    auto v_lo = [&](int s) { return base + (uint32_t)(s * L::SLOT + TC_A_BYTES); };
    auto u_hi = [&](int s) { return base + (uint32_t)(s * L::SLOT + 2 * TC_A_BYTES); };
    auto u_lo = [&](int s) { return base + (uint32_t)(s * L::SLOT + 2 * TC_A_BYTES + L::B_BYTES); };

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_conv + 8 * s, 128);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_tfull + 8 * a, 1);
            mbar_init(bar_tempty + 8 * a, 128);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long total = (long long)p.batches * p.mblocks * p.nblocks;

    if (warp == 0) {
        const bool issuer = elect_one();
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            const int nb = (int)(tile % p.nblocks);
            const int mb = (int)((tile / p.nblocks) % p.mblocks);
            const int xi = (int)(tile / ((long long)p.nblocks * p.mblocks));
            for (int kc = 0; kc < p.kchunks; ++kc) {
                if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, TS_WAIT_EMPTY)) { ok = false; break; }
                if (issuer) {
                    mbar_arrive_expect_tx(bar_full + 8 * stage, TC_A_BYTES + 2 * L::B_BYTES);
                    tma_load_3d(v_hi(stage), &tm_v, bar_full + 8 * stage, kc * TS_KC, mb * TC_BM, xi);
                    tma_load_3d(u_hi(stage), &tm_u, bar_full + 8 * stage, kc * TS_KC, nb * BN, xi);
                    tma_load_3d(u_lo(stage), &tm_u, bar_full + 8 * stage, p.cp + kc * TS_KC, nb * BN, xi);
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
        if (!ok && issuer) drain_after_abort();
    } else if (warp == 1) {
        const bool issuer = elect_one();
        int stage = 0, as = 0;
        uint32_t phase = 0, aphase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            if (!mbar_wait_warp(bar_tempty + 8 * as, aphase ^ 1, abort_flag, p.status, TS_WAIT_TMEM_EMPTY)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN), d_cross = d_tmem + (uint32_t)(2 * BN);
            for (int kc = 0; kc < p.kchunks; ++kc) {
                if (!mbar_wait_warp(bar_conv + 8 * stage, phase, abort_flag, p.status, TS_WAIT_CONVERTED)) { ok = false; break; }
                tc_fence_after();
                const int left = p.cp - kc * TS_KC;     // the last slot of a row may be part empty (and its U heads box reaches into the tails)
                const int ksteps = left >= TS_KC ? TS_KC / TS_UMMA_K : (left + TS_UMMA_K - 1) / TS_UMMA_K;
                const uint64_t vh = smem_desc_k128(v_hi(stage)), vl = smem_desc_k128(v_lo(stage));
                const uint64_t uh = smem_desc_k128(u_hi(stage)), ul = smem_desc_k128(u_lo(stage));
#pragma unroll 4
                for (int ks = 0; ks < ksteps; ++ks)
                    if (issuer) tc_mma<true>(d_cross, vl + (uint64_t)(ks * 2), uh + (uint64_t)(ks * 2), p.idesc, (kc | ks) ? 1u : 0u);
#pragma unroll 4
                for (int ks = 0; ks < ksteps; ++ks)
                    if (issuer) tc_mma<true>(d_cross, vh + (uint64_t)(ks * 2), ul + (uint64_t)(ks * 2), p.idesc, 1u);
#pragma unroll 4
                for (int ks = 0; ks < ksteps; ++ks)
                    if (issuer) tc_mma<true>(d_tmem, vh + (uint64_t)(ks * 2), uh + (uint64_t)(ks * 2), p.idesc, (kc | ks) ? 1u : 0u);
                if (issuer) tc_commit(bar_empty + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
            if (ok && issuer) tc_commit(bar_tfull + 8 * as);
            as ^= 1;
            if (as == 0) aphase ^= 1;
        }
    } else if (warp >= 6) {
        // converters: split the V tile of each slot into heads (in place) and tails
        const int ct = threadIdx.x - 6 * 32;            // 0 .. 127
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            for (int kc = 0; kc < p.kchunks; ++kc) {
                if (!mbar_wait_bounded(bar_full + 8 * stage, phase, abort_flag, p.status, TS_WAIT_FULL)) { ok = false; break; }
                uint4* hi = reinterpret_cast<uint4*>(gen_base + stage * L::SLOT);
                uint4* lo = reinterpret_cast<uint4*>(gen_base + stage * L::SLOT + TC_A_BYTES);
#pragma unroll
                for (int i = 0; i < TC_A_BYTES / 16 / 128; ++i) {
                    const int u = ct + 128 * i;
                    const uint4 raw = hi[u];
                    const tf32x2_t a = split_tf32(__uint_as_float(raw.x)), b = split_tf32(__uint_as_float(raw.y));
                    const tf32x2_t c = split_tf32(__uint_as_float(raw.z)), d = split_tf32(__uint_as_float(raw.w));
                    hi[u] = make_uint4(__float_as_uint(a.hi), __float_as_uint(b.hi), __float_as_uint(c.hi), __float_as_uint(d.hi));
                    lo[u] = make_uint4(__float_as_uint(a.lo), __float_as_uint(b.lo), __float_as_uint(c.lo), __float_as_uint(d.lo));
                }
                fence_async_shared();                   // generic-proxy writes -> visible to the tensor-core (async) proxy
                mbar_arrive(bar_conv + 8 * stage);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        const int quarter = warp % 4;                 // tensor-memory lanes [32*quarter, 32*quarter + 32)
        uint8_t* stage_gen = gen_base + L::STORE_OFF + quarter * 2 * TS_STORE_TILE;
        const uint32_t stage_s = base + L::STORE_OFF + quarter * 2 * TS_STORE_TILE;
        int as = 0;
        uint32_t aphase = 0, issued = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            const int nb = (int)(tile % p.nblocks);
            const int mb = (int)((tile / p.nblocks) % p.mblocks);
            const int xi = (int)(tile / ((long long)p.nblocks * p.mblocks));
            if (!mbar_wait_bounded(bar_tfull + 8 * as, aphase, abort_flag, p.status, TS_WAIT_TMEM_FULL)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const long long row0 = (long long)mb * TC_BM + quarter * 32;
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; ++chunk) {
                uint32_t r[32], rc[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * BN + chunk * 32), r);
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((2 + as) * BN + chunk * 32), rc);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) + __uint_as_float(rc[i]));
                if (chunk == BN / 32 - 1) {           // the accumulator is in registers: hand it back to the MMA warp
                    tc_fence_before();
                    mbar_arrive(bar_tempty + 8 * as);
                }
                const int col0 = nb * BN + chunk * 32;
                if (row0 < p.t_rows && col0 < p.kq) {
                    const uint32_t buf = issued & 1;
                    if (issued >= 2) {                // the store that last used this staging tile must have read it
                        if (lane == 0) tma_store_wait_read<1>();
                        __syncwarp();
                    }
                    float4* dst = reinterpret_cast<float4*>(stage_gen + buf * TS_STORE_TILE + lane * 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        dst[j ^ (lane & 7)] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    fence_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&tm_m, stage_s + buf * TS_STORE_TILE, col0, (int)row0, xi);
                        tma_store_commit();
                    }
                    ++issued;
                }
            }
            as ^= 1;
            if (as == 0) aphase ^= 1;
        }
        if (lane == 0) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int BN, int STAGES>
int run(const CUtensorMap& tm_v, const CUtensorMap& tm_u, const CUtensorMap& tm_m, const TsParams& p, cudaStream_t st) {
    using L = TsSmem<BN, STAGES>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA exceeded");
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(gemm_tc_split_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    WINO_CUDA_CHECK(attr_err);
    const long long total = (long long)p.batches * p.mblocks * p.nblocks;
    const int grid = (int)(total < sm_count() ? total : sm_count());
    ProfScope prof(STAGE_GEMM, st);
    count_launch();
    gemm_tc_split_kernel<BN, STAGES><<<grid, TS_THREADS, L::TOTAL, st>>>(tm_v, tm_u, tm_m, p);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace

int launch_gemm_tc_split(const float* v, const float* u, float* m, int batches, long long t_rows, long long tp, int k,
                         int cp, int kq, cudaStream_t st) {
    if (t_rows <= 0) return WINO_OK;
    if (cp % 4 != 0 || kq % 4 != 0) return fail(WINO_E_BADARG, "gemm_tc_split: row pitch must be a multiple of 16 bytes");
    if (((uintptr_t)v | (uintptr_t)u | (uintptr_t)m) & 15) return fail(WINO_E_BADARG, "gemm_tc_split: buffers must be 16-byte aligned");
    const int bn = k <= 64 ? 64 : 128;
    CUtensorMap tm_v, tm_u, tm_m;
    int rc;
    if ((rc = make_map_k128(&tm_v, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, v, cp, t_rows, tp, batches, TC_BM))) return rc;
    if ((rc = make_map_k128(&tm_u, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, u, 2 * cp, k, k, batches, bn))) return rc;
    if ((rc = make_map_k128(&tm_m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, m, kq, t_rows, tp, batches, 32))) return rc;
    TsParams p;
    p.t_rows = t_rows; p.cp = cp; p.kq = kq; p.batches = batches;
    p.mblocks = (int)((t_rows + TC_BM - 1) / TC_BM);
    p.nblocks = (k + bn - 1) / bn;
    p.kchunks = (cp + TS_KC - 1) / TS_KC;
    p.idesc = make_idesc(OP_TF32, bn);
    if ((rc = status_word(&p.status))) return rc;
    return bn == 64 ? run<64, 4>(tm_v, tm_u, tm_m, p, st) : run<128, 3>(tm_v, tm_u, tm_m, p, st);
}

}  // namespace wino

// Tensor-core batched tile GEMM for sm_100a:  M[xi][t][k] = sum_c V[xi][t][c] * U[xi][k][c].
//
// Takes the role of GEMM_batch_256_128x128_KMKN / _MKNK (comparison/GEMM.cuh:124-255, :4-122) for the TF32 and
// BF16/FP16-operand variants.  The a*a independent GEMMs of the Winograd domain are one persistent launch:
//
//   * work unit = (xi, 128-tile row block, BN-filter column block); CTAs walk the list round-robin with
//     the column block fastest, so CTAs running side by side share the same V tile through L2;
//   * warp 0, one lane: TMA producer.  cp.async.bulk.tensor.3d boxes of 128 rows x 128 bytes (V) and
//     BN rows x 128 bytes (U) land in a STAGES-deep ring of 128B-swizzled shared-memory tiles; rows past
//     the tile / filter count and channels past Cp are zero filled by the TMA unit, so no padding passes;
//   * warp 1, one lane: issues tcgen05.mma (cta_group::1, M = 128, N = BN, K = 32 bytes per instruction)
//     from shared-memory matrix descriptors into one of two FP32 accumulators in tensor memory and
//     commits each ring slot / accumulator to an mbarrier;
//   * warps 2-5: epilogue.  Each warp owns 32 accumulator lanes (= 32 tile rows): tcgen05.ld brings 32
//     columns into registers, the warp lays them out as a 32 x 32 float tile (128-byte swizzled, so the
//     16-byte shared stores are conflict free) in its own double-buffered staging area, and one lane sends
//     it to M with a TMA store (cp.async.bulk.tensor, bulk_group) that writes full 128-byte rows and clips
//     rows past the tile count and columns past Kq.  The accumulator is released as soon as its last
//     column chunk is in registers, so the next unit's MMAs run underneath the stores.
// No TMA multicast, no clusters.  Every mbarrier wait is bounded (2 s of %globaltimer): a wait that gives
// up records its code in a status word, raises a CTA-wide abort flag so the other roles leave their loops
// too, and the CTA frees its tensor memory and returns.
// Bound: 2*a*a*T*C*K flops against a*a*T*(Cp*s + Kq*4) bytes: C/2 flop per byte of M written, so the tensor
// pipe bounds it only for C >= 512; below that it is bound by writing the FP32 products.
#include <cstdlib>
#include <mutex>

#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace wino {

namespace {

constexpr int TC_THREADS = 192;
constexpr int TC_STORE_TILE = 32 * 32 * 4;  // one epilogue staging tile: 32 rows x 32 floats

enum TcWaitCode { TC_WAIT_EMPTY = 1, TC_WAIT_FULL = 2, TC_WAIT_TMEM_EMPTY = 3, TC_WAIT_TMEM_FULL = 4 };

struct TcParams {
    long long t_rows;
    int kq, cp;
    int batches, mblocks, nblocks, kchunks;
    uint32_t idesc;
    int* status;
};

template <int BN, int STAGES>
struct TcSmem {
    static constexpr int B_BYTES = BN * TC_ROW_BYTES;
    static constexpr int RING = STAGES * (TC_A_BYTES + B_BYTES);
    static constexpr int STORE_OFF = RING;               // 4 warps x 2 staging tiles, each 4 KiB (1 KiB aligned)
    static constexpr int BAR_OFF = STORE_OFF + 8 * TC_STORE_TILE;   // full[STAGES], empty[STAGES], tfull[2], tempty[2]
    static constexpr int SLOT_OFF = BAR_OFF + 8 * (2 * STAGES + 4);
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;   // + slack for the 1 KiB alignment of the ring
};

template <int BN, bool TF32, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_u,
               const __grid_constant__ CUtensorMap tm_m, const TcParams p) {
    using L = TcSmem<BN, STAGES>;
    constexpr int ESIZE = TF32 ? 4 : 2;
    constexpr int KC = TC_ROW_BYTES / ESIZE;        // contraction elements per ring slot
    constexpr int UMMA_K = 32 / ESIZE;              // contraction elements per tcgen05.mma
    constexpr uint32_t TMEM_COLS = 2 * BN;          // two accumulators; 128, 256 or 512 columns

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_ring = base, b_ring = base + STAGES * TC_A_BYTES;
    const uint32_t bar_full = base + L::BAR_OFF, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 16;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::SLOT_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::SLOT_OFF + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
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
        {   // the whole warp walks the ring (warp-uniform addresses); one elected lane issues the copies
            const bool issuer = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                const int nb = (int)(tile % p.nblocks);
                const int mb = (int)((tile / p.nblocks) % p.mblocks);
                const int xi = (int)(tile / ((long long)p.nblocks * p.mblocks));
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, TC_WAIT_EMPTY)) { ok = false; break; }
                    if (issuer) {
                        mbar_arrive_expect_tx(bar_full + 8 * stage, TC_A_BYTES + L::B_BYTES);
                        tma_load_3d(a_ring + stage * TC_A_BYTES, &tm_v, bar_full + 8 * stage, kc * KC, mb * TC_BM, xi);
                        tma_load_3d(b_ring + stage * L::B_BYTES, &tm_u, bar_full + 8 * stage, kc * KC, nb * BN, xi);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok && issuer) drain_after_abort();
        }
    } else if (warp == 1) {
        {   // warp-uniform loop, one elected lane issues: from a single-lane branch every tcgen05.mma cost its thread tens of cycles
            const bool issuer = elect_one();
            int stage = 0, as = 0;
            uint32_t phase = 0, aphase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                if (!mbar_wait_warp(bar_tempty + 8 * as, aphase ^ 1, abort_flag, p.status, TC_WAIT_TMEM_EMPTY)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    if (!mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, p.status, TC_WAIT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const int left = p.cp - kc * KC;
                    const int ksteps = left >= KC ? KC / UMMA_K : (left + UMMA_K - 1) / UMMA_K;
                    // descriptors once per ring slot; a K-step adds 32 bytes = 2 sixteen-byte units to the start address
                    const uint64_t a_desc = smem_desc_k128(a_ring + stage * TC_A_BYTES), b_desc = smem_desc_k128(b_ring + stage * L::B_BYTES);
#pragma unroll 4
                    for (int ks = 0; ks < ksteps; ++ks)
                        if (issuer) tc_mma<TF32>(d_tmem, a_desc + (uint64_t)(ks * 2), b_desc + (uint64_t)(ks * 2), p.idesc, (kc | ks) ? 1u : 0u);
                    if (issuer) tc_commit(bar_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok && issuer) tc_commit(bar_tfull + 8 * as);
                as ^= 1;
                if (as == 0) aphase ^= 1;
            }
        }
    } else {
        const int quarter = warp % 4;                 // tensor-memory lanes [32*quarter, 32*quarter + 32)
        uint8_t* stage_gen = gen_base + L::STORE_OFF + quarter * 2 * TC_STORE_TILE;
        const uint32_t stage_s = base + L::STORE_OFF + quarter * 2 * TC_STORE_TILE;
        int as = 0;
        uint32_t aphase = 0, issued = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            const int nb = (int)(tile % p.nblocks);
            const int mb = (int)((tile / p.nblocks) % p.mblocks);
            const int xi = (int)(tile / ((long long)p.nblocks * p.mblocks));
            if (!mbar_wait_bounded(bar_tfull + 8 * as, aphase, abort_flag, p.status, TC_WAIT_TMEM_FULL)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const long long row0 = (long long)mb * TC_BM + quarter * 32;
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; ++chunk) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * BN + chunk * 32), r);
                tmem_ld_wait();
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
                    float4* dst = reinterpret_cast<float4*>(stage_gen + buf * TC_STORE_TILE + lane * 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        dst[j ^ (lane & 7)] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                          __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                    fence_async_shared();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_3d(&tm_m, stage_s + buf * TC_STORE_TILE, col0, (int)row0, xi);
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

// ---- host side ------------------------------------------------------------------------------------------
template <int BN, bool TF32, int STAGES>
int run(const CUtensorMap& tm_v, const CUtensorMap& tm_u, const CUtensorMap& tm_m, const TcParams& p, cudaStream_t st) {
    using L = TcSmem<BN, STAGES>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA exceeded");
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(gemm_tc_kernel<BN, TF32, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    WINO_CUDA_CHECK(attr_err);
    const long long total = (long long)p.batches * p.mblocks * p.nblocks;
    const int grid = (int)(total < sm_count() ? total : sm_count());
    ProfScope prof(STAGE_GEMM, st);
    count_launch();
    gemm_tc_kernel<BN, TF32, STAGES><<<grid, TC_THREADS, L::TOTAL, st>>>(tm_v, tm_u, tm_m, p);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace

int launch_gemm_tc(int operand, const void* v, const void* u, float* m, int batches, long long t_rows, long long tp,
                   int k, int cp, int kq, cudaStream_t st) {
    if (t_rows <= 0) return WINO_OK;
    if (operand != OP_TF32 && operand != OP_BF16 && operand != OP_F16)
        return fail(WINO_E_BADARG, "gemm_tc: bad operand kind %d", operand);
    const int es = operand == OP_TF32 ? 4 : 2;
    if ((cp * es) % 16 != 0 || kq % 4 != 0) return fail(WINO_E_BADARG, "gemm_tc: row pitch must be a multiple of 16 bytes");
    if (((uintptr_t)v | (uintptr_t)u | (uintptr_t)m) & 15) return fail(WINO_E_BADARG, "gemm_tc: buffers must be 16-byte aligned");
    static const int force_bn = [] { const char* e = getenv("WINO_GEMM_BN"); return e ? atoi(e) : 0; }();
    if (!force_bn && gemm_tc_pair_applies(k, cp, t_rows)) return launch_gemm_tc_pair(operand, v, u, m, batches, t_rows, tp, k, cp, kq, st);
    const int bn = force_bn ? force_bn : k <= 64 ? 64 : (k >= 256 && cp >= 512) ? 256 : 128;   // long contractions: wider tiles, fewer passes over V
    const CUtensorMapDataType dt = operand_map_type(operand);
    CUtensorMap tm_v, tm_u, tm_m;
    int rc;
    if ((rc = make_map_k128(&tm_v, dt, es, v, cp, t_rows, tp, batches, TC_BM))) return rc;
    if ((rc = make_map_k128(&tm_u, dt, es, u, cp, k, k, batches, bn))) return rc;
    if ((rc = make_map_k128(&tm_m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, m, kq, t_rows, tp, batches, 32))) return rc;
    TcParams p;
    p.t_rows = t_rows; p.cp = cp; p.kq = kq; p.batches = batches;
    p.mblocks = (int)((t_rows + TC_BM - 1) / TC_BM);
    p.nblocks = (k + bn - 1) / bn;
    p.kchunks = (cp * es + TC_ROW_BYTES - 1) / TC_ROW_BYTES;
    p.idesc = make_idesc(operand, bn);
    if ((rc = status_word(&p.status))) return rc;
    const bool tf32 = operand == OP_TF32;
    if (bn == 256) return tf32 ? run<256, true, 4>(tm_v, tm_u, tm_m, p, st) : run<256, false, 4>(tm_v, tm_u, tm_m, p, st);
    if (bn == 64) return tf32 ? run<64, true, 6>(tm_v, tm_u, tm_m, p, st) : run<64, false, 6>(tm_v, tm_u, tm_m, p, st);
    return tf32 ? run<128, true, 5>(tm_v, tm_u, tm_m, p, st) : run<128, false, 5>(tm_v, tm_u, tm_m, p, st);
}

}  // namespace wino

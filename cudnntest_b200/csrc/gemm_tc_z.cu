// Tensor-core tile GEMM with the first half of the output transform fused into its epilogue (sm_100a).
//
//   Z[i*m + q][t][k] = sum_j ( sum_c V[i*a + j][t][c] * U[i*a + j][k][c] ) * A[j][q]        i < a, q < m = a - 2
//
// i.e. for one row i of the a x a Winograd domain the a products M[i][0..a-1] are reduced to the m values
// (M A)[i][0..m-1] before anything is written.  The reference writes all a*a FP32 products
// (comparison/GEMM.cuh:124-255 into gemmOutput_gpu, read back by wino_invers_*, wrapedConv_NCHW.cuh:1034-1114);
// here 24 instead of 36 values per (tile, filter) leave the SM for F(4x4,3x3) (8 instead of 16 for
// F(2x2,3x3)), and they leave as FP16 when the storage type is BF16: after one 1-D transform (coefficients
// <= 8) FP16 rounding is harmless, where rounding the raw products before the 2-D transform is not.  That cuts
// the product traffic, the dominant HBM term of the whole convolution, by 3x (1.5x for TF32, which keeps FP32).
//
// Structure: as gemm_tc.cu (persistent CTAs, one TMA producer lane, one tcgen05.mma issuing lane, four epilogue
// warps), with these differences:
//   * work unit = (row i of the Winograd domain, 128-tile row block, 64-filter column block): a accumulators
//     of 64 columns each.  Tensor memory is a ring of eight 64-column accumulator slots with a full / empty
//     mbarrier pair per slot, so the MMA lane runs up to 8 - a accumulators ahead of the epilogue;
//   * the epilogue reads the a accumulators 16 columns at a time, applies A^T along j in registers, converts,
//     lays the m result planes out as 128-byte-swizzled 32-row tiles in shared memory and sends each to its Z
//     plane with a TMA store (rows past the tile count and columns past Kq are clipped by the TMA unit).
// All waits are bounded; a wait that gives up raises the CTA's abort flag and records its code.
#include <mutex>

#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "tcgen05.cuh"
#include "wino_math.cuh"

namespace wino {

namespace {

constexpr int TZ_THREADS = 192;
constexpr int TZ_BN = 64;
constexpr int TZ_SLOTS = 512 / TZ_BN;          // accumulator slots in tensor memory
constexpr int TZ_B_BYTES = TZ_BN * TC_ROW_BYTES;
constexpr int TZ_PLANE_TILE = 32 * 128;        // staging tile of one Z plane for one warp: 32 rows x 128 bytes

enum TzWaitCode { TZ_WAIT_EMPTY = 11, TZ_WAIT_FULL = 12, TZ_WAIT_TMEM_EMPTY = 13, TZ_WAIT_TMEM_FULL = 14 };

struct TzParams {
    long long t_rows;
    int kq, cp;
    int mblocks, nblocks, kchunks;
    uint32_t idesc;
    int* status;
};

template <int A, int STAGES>
struct TzSmem {
    static constexpr int M = A - 2;
    static constexpr int RING = STAGES * (TC_A_BYTES + TZ_B_BYTES);
    static constexpr int STORE_OFF = RING;                                  // 4 warps x M planes x 4 KiB
    static constexpr int BAR_OFF = STORE_OFF + 4 * M * TZ_PLANE_TILE;       // full, empty [STAGES]; tfull, tempty [SLOTS]
    static constexpr int SLOT_OFF = BAR_OFF + 8 * (2 * STAGES + 2 * TZ_SLOTS);
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;
};

template <typename ZT>
struct ZPack;
template <>
struct ZPack<float> {   // 16 floats -> four 16-byte chunks
    static constexpr int CHUNKS = 4;
    static __device__ __forceinline__ void pack(const float (&z)[16], uint4 (&out)[4]) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
            out[c] = make_uint4(__float_as_uint(z[4 * c]), __float_as_uint(z[4 * c + 1]), __float_as_uint(z[4 * c + 2]),
                                __float_as_uint(z[4 * c + 3]));
    }
};
template <>
struct ZPack<__half> {  // 16 halves -> two 16-byte chunks
    static constexpr int CHUNKS = 2;
    static __device__ __forceinline__ void pack(const float (&z)[16], uint4 (&out)[2]) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                __half2 h = __floats2half2_rn(z[8 * c + 2 * e], z[8 * c + 2 * e + 1]);
                w[e] = *reinterpret_cast<uint32_t*>(&h);
            }
            out[c] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
};

template <int A, bool TF32, typename ZT, int STAGES>
__global__ void __launch_bounds__(TZ_THREADS, 1)
gemm_tc_z_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_u,
                 const __grid_constant__ CUtensorMap tm_z, const TzParams p) {
    using L = TzSmem<A, STAGES>;
    constexpr int M = A - 2;
    constexpr int ESIZE = TF32 ? 4 : 2;
    constexpr int KC = TC_ROW_BYTES / ESIZE;
    constexpr int UMMA_K = 32 / ESIZE;
    constexpr int SG = 128 / (int)sizeof(ZT);        // columns per store group: one 128-byte row of a Z plane
    constexpr int CHUNKS = ZPack<ZT>::CHUNKS;        // 16-byte chunks per 16 columns

    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t a_ring = base, b_ring = base + STAGES * TC_A_BYTES;
    const uint32_t bar_full = base + L::BAR_OFF, bar_empty = bar_full + 8 * STAGES;
    const uint32_t bar_tfull = bar_empty + 8 * STAGES, bar_tempty = bar_tfull + 8 * TZ_SLOTS;
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen_base + L::SLOT_OFF);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(gen_base + L::SLOT_OFF + 4);

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int s = 0; s < TZ_SLOTS; ++s) {
            mbar_init(bar_tfull + 8 * s, 1);
            mbar_init(bar_tempty + 8 * s, 128);
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long total = (long long)A * p.mblocks * p.nblocks;

    if (warp == 0) {
        {   // the whole warp walks the ring (warp-uniform addresses); one elected lane issues the copies
            const bool issuer = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long unit = blockIdx.x; ok && unit < total; unit += gridDim.x) {
                const int nb = (int)(unit % p.nblocks);
                const int mb = (int)((unit / p.nblocks) % p.mblocks);
                const int i = (int)(unit / ((long long)p.nblocks * p.mblocks));
                for (int j = 0; ok && j < A; ++j) {
                    const int xi = i * A + j;
                    for (int kc = 0; kc < p.kchunks; ++kc) {
                        if (!mbar_wait_warp(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, TZ_WAIT_EMPTY)) { ok = false; break; }
                        if (issuer) {
                            mbar_arrive_expect_tx(bar_full + 8 * stage, TC_A_BYTES + TZ_B_BYTES);
                            tma_load_3d(a_ring + stage * TC_A_BYTES, &tm_v, bar_full + 8 * stage, kc * KC, mb * TC_BM, xi);
                            tma_load_3d(b_ring + stage * TZ_B_BYTES, &tm_u, bar_full + 8 * stage, kc * KC, nb * TZ_BN, xi);
                        }
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
                }
            }
            if (!ok && issuer) drain_after_abort();
        }
    } else if (warp == 1) {
        {   // warp-uniform loop, one elected lane issues: from a single-lane branch every tcgen05.mma cost its thread tens of cycles
            const bool issuer = elect_one();
            int stage = 0;
            uint32_t phase = 0;
            unsigned long long g = 0;   // accumulators produced so far
            bool ok = true;
            for (long long unit = blockIdx.x; ok && unit < total; unit += gridDim.x) {
                for (int j = 0; ok && j < A; ++j, ++g) {
                    const int slot = (int)(g % TZ_SLOTS);
                    const uint32_t sphase = (uint32_t)((g / TZ_SLOTS) & 1);
                    if (!mbar_wait_warp(bar_tempty + 8 * slot, sphase ^ 1, abort_flag, p.status, TZ_WAIT_TMEM_EMPTY)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(slot * TZ_BN);
                    for (int kc = 0; kc < p.kchunks; ++kc) {
                        if (!mbar_wait_warp(bar_full + 8 * stage, phase, abort_flag, p.status, TZ_WAIT_FULL)) { ok = false; break; }
                        tc_fence_after();
                        const int left = p.cp - kc * KC;
                        const int ksteps = left >= KC ? KC / UMMA_K : (left + UMMA_K - 1) / UMMA_K;
                        const uint64_t a_desc = smem_desc_k128(a_ring + stage * TC_A_BYTES), b_desc = smem_desc_k128(b_ring + stage * TZ_B_BYTES);
#pragma unroll 4
                        for (int ks = 0; ks < ksteps; ++ks)
                            if (issuer) tc_mma<TF32>(d_tmem, a_desc + (uint64_t)(ks * 2), b_desc + (uint64_t)(ks * 2), p.idesc, (kc | ks) ? 1u : 0u);
                        if (issuer) tc_commit(bar_empty + 8 * stage);
                        if (++stage == STAGES) { stage = 0; phase ^= 1; }
                    }
                    if (ok && issuer) tc_commit(bar_tfull + 8 * slot);
                }
            }
        }
    } else {
        const int quarter = warp % 4;                 // tensor-memory lanes [32*quarter, 32*quarter + 32)
        uint8_t* stage_gen = gen_base + L::STORE_OFF + quarter * M * TZ_PLANE_TILE;
        const uint32_t stage_s = base + L::STORE_OFF + quarter * M * TZ_PLANE_TILE;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        unsigned long long g = 0;
        bool ok = true, pending = false;
        for (long long unit = blockIdx.x; ok && unit < total; unit += gridDim.x, g += A) {
            const int nb = (int)(unit % p.nblocks);
            const int mb = (int)((unit / p.nblocks) % p.mblocks);
            const int i = (int)(unit / ((long long)p.nblocks * p.mblocks));
#pragma unroll 1
            for (int j = 0; j < A; ++j) {
                const unsigned long long gj = g + j;
                if (ok && !mbar_wait_bounded(bar_tfull + 8 * (int)(gj % TZ_SLOTS), (uint32_t)((gj / TZ_SLOTS) & 1), abort_flag,
                                             p.status, TZ_WAIT_TMEM_FULL))
                    ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const long long row0 = (long long)mb * TC_BM + quarter * 32;
#pragma unroll 1
            for (int sg = 0; sg < TZ_BN / SG; ++sg) {
                if (pending) {                        // the previous stores must have read the staging tiles
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
                    pending = false;
                }
#pragma unroll 1
                for (int c16 = 0; c16 < SG / 16; ++c16) {
                    const int col = sg * SG + c16 * 16;
                    uint32_t r[A][16];
#pragma unroll
                    for (int j = 0; j < A; ++j)
                        tmem_ld_32x16(lane_addr + (uint32_t)(((g + j) % TZ_SLOTS) * TZ_BN + col), r[j]);
                    tmem_ld_wait();
                    if (sg == TZ_BN / SG - 1 && c16 == SG / 16 - 1) {   // all a accumulators are in registers
                        tc_fence_before();
#pragma unroll
                        for (int j = 0; j < A; ++j) mbar_arrive(bar_tempty + 8 * (int)((g + j) % TZ_SLOTS));
                    }
                    float z[M][16];
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        float mj[A], zq[M];
#pragma unroll
                        for (int j = 0; j < A; ++j) mj[j] = __uint_as_float(r[j][e]);
                        at_1d<A>(mj, zq);
#pragma unroll
                        for (int q = 0; q < M; ++q) z[q][e] = zq[q];
                    }
#pragma unroll
                    for (int q = 0; q < M; ++q) {
                        uint4 packed[CHUNKS];
                        ZPack<ZT>::pack(z[q], packed);
                        uint4* dst = reinterpret_cast<uint4*>(stage_gen + q * TZ_PLANE_TILE + lane * 128);
#pragma unroll
                        for (int c = 0; c < CHUNKS; ++c) dst[(c16 * CHUNKS + c) ^ (lane & 7)] = packed[c];
                    }
                }
                const int col0 = nb * TZ_BN + sg * SG;
                fence_async_shared();
                __syncwarp();
                if (row0 < p.t_rows && col0 < p.kq) {
                    if (lane == 0) {
#pragma unroll
                        for (int q = 0; q < M; ++q) tma_store_3d(&tm_z, stage_s + q * TZ_PLANE_TILE, col0, (int)row0, i * M + q);
                        tma_store_commit();
                    }
                    pending = true;
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int A, bool TF32, typename ZT, int STAGES>
int run(const CUtensorMap& tm_v, const CUtensorMap& tm_u, const CUtensorMap& tm_z, const TzParams& p, cudaStream_t st) {
    using L = TzSmem<A, STAGES>;
    static_assert(L::TOTAL <= 232448, "shared memory budget of one CTA exceeded");
    static std::once_flag once[64];
    int dev = 0;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    cudaError_t attr_err = cudaSuccess;
    std::call_once(once[dev & 63], [&] {
        attr_err = cudaFuncSetAttribute(gemm_tc_z_kernel<A, TF32, ZT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    });
    WINO_CUDA_CHECK(attr_err);
    const long long total = (long long)A * p.mblocks * p.nblocks;
    const int grid = (int)(total < sm_count() ? total : sm_count());
    ProfScope prof(STAGE_GEMM_ROWFUSED, st);
    count_launch();
    gemm_tc_z_kernel<A, TF32, ZT, STAGES><<<grid, TZ_THREADS, L::TOTAL, st>>>(tm_v, tm_u, tm_z, p);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace

int launch_gemm_tc_z(int operand, int a, const void* v, const void* u, void* z, long long t_rows, long long tp, int k, int cp,
                     int kq, cudaStream_t st) {
    if (t_rows <= 0) return WINO_OK;
    if (operand != OP_TF32 && operand != OP_BF16 && operand != OP_F16)
        return fail(WINO_E_BADARG, "gemm_tc_z: bad operand kind %d", operand);
    if (a != 4 && a != 6) return fail(WINO_E_BADARG, "gemm_tc_z: bad tile side %d", a);
    const int es = operand == OP_TF32 ? 4 : 2;
    const int zs = operand == OP_TF32 ? 4 : 2;
    if ((cp * es) % 16 != 0 || (kq * zs) % 16 != 0) return fail(WINO_E_BADARG, "gemm_tc_z: row pitch must be a multiple of 16 bytes");
    if (((uintptr_t)v | (uintptr_t)u | (uintptr_t)z) & 15) return fail(WINO_E_BADARG, "gemm_tc_z: buffers must be 16-byte aligned");
    const CUtensorMapDataType dt = operand_map_type(operand);
    CUtensorMap tm_v, tm_u, tm_z;
    int rc;
    if ((rc = make_map_k128(&tm_v, dt, es, v, cp, t_rows, tp, a * a, TC_BM))) return rc;
    if ((rc = make_map_k128(&tm_u, dt, es, u, cp, k, k, a * a, TZ_BN))) return rc;
    if ((rc = make_map_k128(&tm_z, zs == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, zs, z, kq, t_rows, tp,
                            a * (a - 2), 32)))
        return rc;
    TzParams p;
    p.t_rows = t_rows; p.cp = cp; p.kq = kq;
    p.mblocks = (int)((t_rows + TC_BM - 1) / TC_BM);
    p.nblocks = (k + TZ_BN - 1) / TZ_BN;
    p.kchunks = (cp * es + TC_ROW_BYTES - 1) / TC_ROW_BYTES;
    p.idesc = make_idesc(operand, TZ_BN);
    if ((rc = status_word(&p.status))) return rc;
    if (operand == OP_TF32)
        return a == 6 ? run<6, true, float, 5>(tm_v, tm_u, tm_z, p, st) : run<4, true, float, 6>(tm_v, tm_u, tm_z, p, st);
    return a == 6 ? run<6, false, __half, 5>(tm_v, tm_u, tm_z, p, st) : run<4, false, __half, 6>(tm_v, tm_u, tm_z, p, st);
}

}  // namespace wino

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
//   * warps 2-5: epilogue.  Each thread owns one accumulator lane (= one tile row), reads it with
//     tcgen05.ld 32 columns at a time and stores 128-byte row segments of M; the second accumulator lets
//     the next unit's MMAs run underneath.
// No TMA multicast, no clusters.  Every mbarrier wait is bounded (2 s of %globaltimer): a wait that gives
// up records its code in a status word, raises a CTA-wide abort flag so the other roles leave their loops
// too, and the CTA frees its tensor memory and returns.
// Bound: the tensor pipe for large C; for C <= 256 the FP32 product buffer written by the epilogue
// (4*kq bytes per 2*cp MACs) makes it memory bound, which is why slabs are kept L2 resident.
#include <cuda.h>

#include <mutex>

#include "gemm_tc.cuh"

namespace wino {

__device__ int g_tc_status = 0;

namespace {

constexpr int TC_BM = 128;
constexpr int TC_ROW_BYTES = 128;           // bytes of contraction dimension per ring slot row (one swizzle span)
constexpr int TC_A_BYTES = TC_BM * TC_ROW_BYTES;
constexpr int TC_THREADS = 192;
constexpr unsigned long long TC_WAIT_NS = 2000000000ull;

enum TcWaitCode { TC_WAIT_EMPTY = 1, TC_WAIT_FULL = 2, TC_WAIT_TMEM_EMPTY = 3, TC_WAIT_TMEM_FULL = 4 };

struct TcParams {
    float* m;
    long long t_rows, tp;
    int k, cp, kq, batches;
    int mblocks, nblocks, kchunks;
    uint32_t idesc;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Bounded wait.  Returns false if the CTA is aborting or the wait ran out of time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 0xff) == 0xff) {
            if (*abort_flag) return false;
            const unsigned long long now = global_timer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > TC_WAIT_NS) {
                *abort_flag = 1;
                atomicCAS(&g_tc_status, 0, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// mbarrier arrive once every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart, 8-row groups
// 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                    // descriptor version for tcgen05
    d |= (uint64_t)2 << 61;                    // 128-byte swizzle
    return d;
}

template <bool TF32>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if (TF32) {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "setp.ne.b32 p, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
            "}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// 32 lanes x 32 consecutive 32-bit columns of tensor memory -> 32 registers per thread
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int BN, int STAGES>
struct TcSmem {
    static constexpr int B_BYTES = BN * TC_ROW_BYTES;
    static constexpr int RING = STAGES * (TC_A_BYTES + B_BYTES);
    static constexpr int BAR_OFF = RING;                 // full[STAGES], empty[STAGES], tfull[2], tempty[2]
    static constexpr int SLOT_OFF = BAR_OFF + 8 * (2 * STAGES + 4);
    static constexpr int TOTAL = SLOT_OFF + 16 + 1024;   // + slack for the 1 KiB alignment of the ring
};

template <int BN, bool TF32, int STAGES>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_u, const TcParams p) {
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
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const long long total = (long long)p.batches * p.mblocks * p.nblocks;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                const int nb = (int)(tile % p.nblocks);
                const int mb = (int)((tile / p.nblocks) % p.mblocks);
                const int xi = (int)(tile / ((long long)p.nblocks * p.mblocks));
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, TC_WAIT_EMPTY)) { ok = false; break; }
                    mbar_arrive_expect_tx(bar_full + 8 * stage, TC_A_BYTES + L::B_BYTES);
                    tma_load_3d(a_ring + stage * TC_A_BYTES, &tm_v, bar_full + 8 * stage, kc * KC, mb * TC_BM, xi);
                    tma_load_3d(b_ring + stage * L::B_BYTES, &tm_u, bar_full + 8 * stage, kc * KC, nb * BN, xi);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            if (!ok) {
                // copies already issued may still be landing in this CTA's shared memory: give them time
                const unsigned long long t0 = global_timer();
                while (global_timer() - t0 < 1000000ull) __nanosleep(1000);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int stage = 0, as = 0;
            uint32_t phase = 0, aphase = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
                if (!mbar_wait(bar_tempty + 8 * as, aphase ^ 1, abort_flag, TC_WAIT_TMEM_EMPTY)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
                for (int kc = 0; kc < p.kchunks; ++kc) {
                    if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag, TC_WAIT_FULL)) { ok = false; break; }
                    tc_fence_after();
                    const int left = p.cp - kc * KC;
                    const int ksteps = left >= KC ? KC / UMMA_K : (left + UMMA_K - 1) / UMMA_K;
                    const uint32_t a_s = a_ring + stage * TC_A_BYTES, b_s = b_ring + stage * L::B_BYTES;
                    for (int ks = 0; ks < ksteps; ++ks)
                        tc_mma<TF32>(d_tmem, smem_desc_k128(a_s + ks * 32), smem_desc_k128(b_s + ks * 32), p.idesc,
                                     (kc | ks) ? 1u : 0u);
                    tc_commit(bar_empty + 8 * stage);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) tc_commit(bar_tfull + 8 * as);
                as ^= 1;
                if (as == 0) aphase ^= 1;
            }
        }
    } else {
        const int quarter = warp % 4;                 // tensor-memory lanes [32*quarter, 32*quarter + 32)
        const int row_in_tile = quarter * 32 + lane;
        int as = 0;
        uint32_t aphase = 0;
        bool ok = true;
        for (long long tile = blockIdx.x; ok && tile < total; tile += gridDim.x) {
            const int nb = (int)(tile % p.nblocks);
            const int mb = (int)((tile / p.nblocks) % p.mblocks);
            const int xi = (int)(tile / ((long long)p.nblocks * p.mblocks));
            if (!mbar_wait(bar_tfull + 8 * as, aphase, abort_flag, TC_WAIT_TMEM_FULL)) ok = false;
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const long long row = (long long)mb * TC_BM + row_in_tile;
            float* dst = p.m + ((long long)xi * p.tp + row) * p.kq;
#pragma unroll 1
            for (int chunk = 0; chunk < BN / 32; ++chunk) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * BN + chunk * 32), r);
                tmem_ld_wait();
                const int col0 = nb * BN + chunk * 32;
                if (row < p.t_rows) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (col0 + 4 * j < p.kq)
                            *reinterpret_cast<float4*>(dst + col0 + 4 * j) =
                                make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                            __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty + 8 * as);
            as ^= 1;
            if (as == 0) aphase ^= 1;
        }
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// 3-D map over [batches][rows][cp] (cp contiguous); box = 128 bytes x box_rows x 1, 128-byte swizzle
int make_map(CUtensorMap* map, int operand, const void* ptr, int cp, long long rows, long long row_pitch, int batches,
             int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(WINO_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
    const int es = operand == OP_TF32 ? 4 : 2;
    const CUtensorMapDataType dt = operand == OP_TF32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : operand == OP_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    cuuint64_t dims[3] = {(cuuint64_t)cp, (cuuint64_t)rows, (cuuint64_t)batches};
    cuuint64_t strides[2] = {(cuuint64_t)cp * es, (cuuint64_t)row_pitch * cp * es};
    cuuint32_t box[3] = {(cuuint32_t)(TC_ROW_BYTES / es), (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WINO_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return WINO_OK;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

uint32_t make_idesc(int operand, int bn) {
    const uint32_t fmt = operand == OP_TF32 ? 2u : operand == OP_BF16 ? 1u : 0u;  // kind::f16: 0 = F16, 1 = BF16
    uint32_t d = 0;
    d |= 1u << 4;                      // accumulator format: F32
    d |= fmt << 7;                     // A format
    d |= fmt << 10;                    // B format
    /* bits 13, 14: no negation; bits 15, 16: A and B are K-major */
    d |= (uint32_t)(bn >> 3) << 17;    // N / 8
    d |= (uint32_t)(TC_BM >> 4) << 24; // M / 16
    return d;
}

template <int BN, bool TF32, int STAGES>
int run(const CUtensorMap& tm_v, const CUtensorMap& tm_u, const TcParams& p, cudaStream_t st) {
    using L = TcSmem<BN, STAGES>;
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
    gemm_tc_kernel<BN, TF32, STAGES><<<grid, TC_THREADS, L::TOTAL, st>>>(tm_v, tm_u, p);
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
    const int bn = k <= 64 ? 64 : 128;
    CUtensorMap tm_v, tm_u;
    int rc;
    if ((rc = make_map(&tm_v, operand, v, cp, t_rows, tp, batches, TC_BM))) return rc;
    if ((rc = make_map(&tm_u, operand, u, cp, k, k, batches, bn))) return rc;
    TcParams p;
    p.m = m; p.t_rows = t_rows; p.tp = tp; p.k = k; p.cp = cp; p.kq = kq; p.batches = batches;
    p.mblocks = (int)((t_rows + TC_BM - 1) / TC_BM);
    p.nblocks = (k + bn - 1) / bn;
    p.kchunks = (cp * es + TC_ROW_BYTES - 1) / TC_ROW_BYTES;
    p.idesc = make_idesc(operand, bn);
    const bool tf32 = operand == OP_TF32;
    if (bn == 64) return tf32 ? run<64, true, 8>(tm_v, tm_u, p, st) : run<64, false, 8>(tm_v, tm_u, p, st);
    return tf32 ? run<128, true, 6>(tm_v, tm_u, p, st) : run<128, false, 6>(tm_v, tm_u, p, st);
}

int read_and_clear_tc_status(int* status) {
    WINO_CUDA_CHECK(cudaDeviceSynchronize());
    int s = 0;
    WINO_CUDA_CHECK(cudaMemcpyFromSymbol(&s, g_tc_status, sizeof(int)));
    if (s != 0) {
        const int zero = 0;
        WINO_CUDA_CHECK(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
    }
    *status = s;
    return WINO_OK;
}

}  // namespace wino

// Exact-FP32 batched tile GEMM:  M[xi][t][k] = sum_c V[xi][t][c] * U[xi][k][c]   for xi in [0, a*a).
//
// Replaces GEMM_batch_256_128x128_KMKN / _MKNK (comparison/GEMM.cuh:124-255, :4-122) for the variant that
// keeps the reference's FP32 FFMA arithmetic.  Same blocking idea (128 x BN block, 8- or 16-deep k slices,
// 256 threads, 8 x (BN/16) register micro-tile as 4x4 quadrants, double-buffered shared memory with
// register prefetch), written for the K-major operand buffers this library uses: both operands have the
// contraction index contiguous, so a thread fetches one float4 along c and scatters it into a
// [k][row] shared tile whose pitch (BM + 4) keeps the transposing stores conflict free.
// Rows beyond the tile count / filter count are predicated (zero loads, skipped stores); the reference
// kernel has no bounds checks and needs M, N multiples of 128.
// Bound: FP32 FFMA issue rate (2 * a*a * T * C * K flops), not memory.
#include <cstdlib>

#include "common.cuh"

namespace wino {

constexpr int GF_BM = 128;

// GF_BK: depth of a shared-memory slice.  16 halves the block-wide barriers per flop (128-filter blocks: 47.8 -> 52.3
// TFLOP/s at C = K = 512); the 64-filter variant keeps 8, where its smaller register count lets three CTAs share an SM.
template <int BN, int GF_BK>
__global__ void __launch_bounds__(256, BN == 64 ? 3 : 2) gemm_ffma_kernel(const float* __restrict__ V, const float* __restrict__ U,
                                                        float* __restrict__ Mo, long long t_rows, long long tp, int K,
                                                        int cp, int kq) {
    constexpr int TN = BN / 16;         // columns per thread: 8 (two quadrants) or 4 (one)
    constexpr int NQ = TN / 4;          // column quadrants
    constexpr int KQ = GF_BK / 4;                      // float4 per row of a slice
    constexpr int PASS_ROWS = 256 / KQ;                // rows one pass of the 256 threads covers: 64 or 128
    constexpr int A_U = GF_BM / PASS_ROWS;             // passes over the V tile: 2 or 1
    constexpr int B_U = BN >= PASS_ROWS ? BN / PASS_ROWS : 1;   // passes over the U tile (threads beyond a narrow tile idle)
    __shared__ __align__(16) float As[2][GF_BK][GF_BM + 4];
    __shared__ __align__(16) float Bs[2][GF_BK][BN + 4];

    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const long long m0 = (long long)blockIdx.x * GF_BM;
    const int n0 = blockIdx.y * BN;
    const int xi = blockIdx.z;
    const float* Ap = V + (long long)xi * tp * cp;
    const float* Bp = U + (long long)xi * K * cp;
    float* Cp = Mo + (long long)xi * tp * kq;

    // global -> register staging: a slice of a tile is 128 (or BN) rows of KQ float4; a thread stages the float4 at
    // contraction offset lk of row lrow + PASS_ROWS u, one pass per GF_BK / A_U k-steps so that only one pass's
    // registers are live at a time
    const int lrow = tid / KQ, lk = (tid % KQ) * 4;
    const bool b_act = lrow < BN;
    const float* a_src = Ap + (m0 + lrow) * cp + lk;
    const float* b_src = Bp + (long long)(n0 + lrow) * cp + lk;
    const long long half_step = (long long)PASS_ROWS * cp;
    const long long a_left = t_rows - m0 - lrow;          // row lrow + PASS_ROWS u exists iff PASS_ROWS u < a_left
    const int b_left = K - n0 - lrow;

    // accumulators as float2 pairs of adjacent columns: one fma.rn.f32x2 (two exact FP32 FMAs, same rounding as two
    // FFMAs) per pair halves the issue slots the multiply-adds take (measured: 41.8 -> 47.8 TFLOP/s at C = K = 512).
    // Tried and dropped: a V tile stored with doubled values to save the register moves that build {a, a} (the extra
    // shared-memory reads cost more: 35.7 TFLOP/s).
    float2 acc[8][TN / 2];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < TN / 2; ++j) acc[i][j] = make_float2(0.f, 0.f);

    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 ra, rb;
    // half u of slice ks into registers (zero beyond the tile, the filter count and the contraction length)
    auto fetch = [&](int ks, int u) {
        const bool k_ok = ks * GF_BK + lk + 4 <= cp;
        ra = (k_ok && PASS_ROWS * u < a_left) ? __ldg(reinterpret_cast<const float4*>(a_src + u * half_step + ks * GF_BK)) : zero4;
        if (u < B_U) rb = (k_ok && b_act && PASS_ROWS * u < b_left) ? __ldg(reinterpret_cast<const float4*>(b_src + u * half_step + ks * GF_BK)) : zero4;
    };
    auto stash = [&](int buf, int u) {
        const int r = lrow + PASS_ROWS * u;
        As[buf][lk + 0][r] = ra.x; As[buf][lk + 1][r] = ra.y; As[buf][lk + 2][r] = ra.z; As[buf][lk + 3][r] = ra.w;
        if (u < B_U && b_act) { Bs[buf][lk + 0][r] = rb.x; Bs[buf][lk + 1][r] = rb.y; Bs[buf][lk + 2][r] = rb.z; Bs[buf][lk + 3][r] = rb.w; }
    };
#pragma unroll
    for (int u = 0; u < A_U; ++u) { fetch(0, u); stash(0, u); }
    __syncthreads();

    const int ksteps = (cp + GF_BK - 1) / GF_BK;  // cp is a multiple of 8: the last slice may be half empty (zeros)
    for (int ks = 0; ks < ksteps; ++ks) {
        const int cur = ks & 1;
        const bool more = ks + 1 < ksteps;
#pragma unroll
        for (int kk = 0; kk < GF_BK; ++kk) {
            if (kk == 0 && more) fetch(ks + 1, 0);
            if (A_U == 2 && kk == GF_BK / 2 && more) { stash(cur ^ 1, 0); fetch(ks + 1, 1); }
            float a[8], b[TN];
            const float4 a0 = *reinterpret_cast<const float4*>(&As[cur][kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[cur][kk][64 + ty * 4]);
            a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
            a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const float4 bq = *reinterpret_cast<const float4*>(&Bs[cur][kk][q * (BN / 2) + tx * 4]);
                b[q * 4 + 0] = bq.x; b[q * 4 + 1] = bq.y; b[q * 4 + 2] = bq.z; b[q * 4 + 3] = bq.w;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 ai = make_float2(a[i], a[i]);
#pragma unroll
                for (int j = 0; j < TN / 2; ++j) acc[i][j] = __ffma2_rn(ai, make_float2(b[2 * j], b[2 * j + 1]), acc[i][j]);
            }
        }
        if (more) stash(cur ^ 1, A_U - 1);
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const long long row = m0 + (i / 4) * 64 + ty * 4 + (i % 4);
        if (row >= t_rows) continue;
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
            const int col = n0 + q * (BN / 2) + tx * 4;
            if (col < kq)  // kq is a multiple of 8 >= K; columns in [K, kq) hold zeros (U rows beyond K load as zero)
                *reinterpret_cast<float4*>(Cp + row * kq + col) =
                    make_float4(acc[i][q * 2].x, acc[i][q * 2].y, acc[i][q * 2 + 1].x, acc[i][q * 2 + 1].y);
        }
    }
}

int launch_gemm_ffma(const float* v, const float* u, float* m, int batches, long long t_rows, long long tp, int k,
                     int cp, int kq, cudaStream_t st) {
    if (t_rows <= 0) return WINO_OK;
    if (cp % 8 != 0 || kq % 4 != 0) return fail(WINO_E_BADARG, "gemm_ffma: cp=%d must be a multiple of 8, kq=%d of 4", cp, kq);
    const unsigned mb = (unsigned)((t_rows + GF_BM - 1) / GF_BM);
    ProfScope prof(STAGE_GEMM, st);
    count_launch();
    static const int force_bn = [] { const char* e = getenv("WINO_FFMA_BN"); return e ? atoi(e) : 0; }();
    if (force_bn ? force_bn == 64 : k <= 64) {
        dim3 grid(mb, (unsigned)((k + 63) / 64), (unsigned)batches);
        gemm_ffma_kernel<64, 8><<<grid, 256, 0, st>>>(v, u, m, t_rows, tp, k, cp, kq);
    } else {
        dim3 grid(mb, (unsigned)((k + 127) / 128), (unsigned)batches);
        gemm_ffma_kernel<128, 16><<<grid, 256, 0, st>>>(v, u, m, t_rows, tp, k, cp, kq);
    }
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace wino

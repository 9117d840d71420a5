// Tensor-core batched tile GEMM (tcgen05 / TMEM / TMA), declarations.
#pragma once

#include "common.cuh"

namespace wino {

// M[xi][t][k] = sum_c V[xi][t][c] * U[xi][k][c], xi in [0, batches); operand = OP_TF32 / OP_BF16 / OP_F16.
// V: [batches][tp][cp], U: [batches][k][cp] (cp elements per row, row pitch a multiple of 16 bytes),
// M: [batches][tp][kq] float.  Rows t >= t_rows are neither read nor written.
int launch_gemm_tc(int operand, const void* v, const void* u, float* m, int batches, long long t_rows, long long tp,
                   int k, int cp, int kq, cudaStream_t st);

// The same product on CTA pairs (tcgen05.mma.cta_group::2, 256 tiles x 256 filters per pair): gemm_tc_pair.cu.
// launch_gemm_tc forwards to it where gemm_tc_pair_applies (wide layers; WINO_GEMM_PAIR = 0 / 1 / 2 overrides).
bool gemm_tc_pair_applies(int k, int cp, long long t_rows);
int launch_gemm_tc_pair(int operand, const void* v, const void* u, float* m, int batches, long long t_rows, long long tp,
                        int k, int cp, int kq, cudaStream_t st, bool m24 = false);
// 3-byte products (upper 24 bits of each float, as a 16-bit plane and a byte plane): where the pair kernel applies,
// WINO_M24=0 disables
bool gemm_tc_m24_applies(int operand, int k, int cp, int kq, long long t_rows);

// Split-TF32 variant (FP32X3): V plain FP32 rows of cp floats, U rows of 2*cp floats (cp TF32 heads, then cp TF32 tails);
// M = lo(V)*hi(U) + hi(V)*lo(U) + hi(V)*hi(U) with V split inside the kernel (gemm_tc_split.cu).
int launch_gemm_tc_split(const float* v, const float* u, float* m, int batches, long long t_rows, long long tp, int k,
                         int cp, int kq, cudaStream_t st);

// Row-fused variant: Z[i*m + q][t][k] = sum_j M[i*a + j][t][k] * A[j][q]; Z is float for OP_TF32, half otherwise.
// V, U as above with a*a batches; Z: [a*m][tp][kq].
int launch_gemm_tc_z(int operand, int a, const void* v, const void* u, void* z, long long t_rows, long long tp, int k, int cp,
                     int kq, cudaStream_t st);

}  // namespace wino

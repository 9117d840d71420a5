// Tensor-core batched tile GEMM (tcgen05 / TMEM / TMA), declarations.
#pragma once

#include "common.cuh"

namespace wino {

// M[xi][t][k] = sum_c V[xi][t][c] * U[xi][k][c], xi in [0, batches); operand = OP_TF32 / OP_BF16 / OP_F16.
// V: [batches][tp][cp], U: [batches][k][cp] (cp elements per row, row pitch a multiple of 16 bytes),
// M: [batches][tp][kq] float.  Rows t >= t_rows are neither read nor written.
// operand = OP_TF32X3: V and U rows hold 2*cp floats, cp TF32 heads followed by cp TF32 tails, and
// M = V_lo * U_hi + V_hi * U_lo + V_hi * U_hi (three TF32 passes over the contraction in one accumulator).
int launch_gemm_tc(int operand, const void* v, const void* u, float* m, int batches, long long t_rows, long long tp,
                   int k, int cp, int kq, cudaStream_t st);

// Row-fused variant: Z[i*m + q][t][k] = sum_j M[i*a + j][t][k] * A[j][q]; Z is float for OP_TF32, half otherwise.
// V, U as above with a*a batches; Z: [a*m][tp][kq].
int launch_gemm_tc_z(int operand, int a, const void* v, const void* u, void* z, long long t_rows, long long tp, int k, int cp,
                     int kq, cudaStream_t st);

}  // namespace wino

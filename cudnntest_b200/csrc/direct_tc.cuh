// Shared between the single-CTA and the CTA-pair direct convolution kernels (direct_tc.cu, direct_tc2.cu).
#pragma once

#include "common.cuh"

namespace wino {

constexpr int DT_TW = 8, DT_TH = 16;                 // output tile
constexpr int DT_BOX_W = DT_TW + 2, DT_BOX_H = DT_TH + 2;   // halo box: 10 x 18 pixels
constexpr int DT_A_BYTES = DT_BOX_W * DT_BOX_H * 128;                      // bytes one halo box brings in
constexpr int DT_A_STRIDE = (DT_A_BYTES + 1023) / 1024 * 1024;            // ring slots stay 1 KiB aligned
constexpr int DT_EPI_WARPS = 8;                      // two warps per tensor-memory lane quarter, each takes half the filter columns
constexpr int DT_THREADS = 64 + 32 * DT_EPI_WARPS;

enum DtWaitCode { DT_W_A_EMPTY = 41, DT_W_A_FULL = 42, DT_W_B_EMPTY = 43, DT_W_B_FULL = 44, DT_W_T_EMPTY = 45, DT_W_T_FULL = 46,
                  DT_W_B_RESIDENT = 47 };

struct DtParams {
    const float* bias;
    void* y;                     // bfloat16 (BF16 variant) or float (TF32 variant)
    int N, OH, OW, K, pad;
    int PH, PW;                  // stored output size (after the optional pool)
    int tiles_x, tiles_y, nblocks, cchunks;
    int relu, pool;
    int y_nchw;                  // filters-as-M kernel only: y is stored NCHW (pixels contiguous) instead of NHWC
    uint32_t idesc;
    int* status;
};

// CTA-pair kernel (direct_tc2.cu); same packed filters and tensor maps as the single-CTA kernel
bool direct_tc2_applies(const wino_conv_desc& d);
int launch_direct_tc2(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                      cudaStream_t st, bool y_nchw = false);

// CTA-pair kernel with the filters as the M operand, K >= 256 (direct_tc2t.cu)
bool direct_tc2t_applies(const wino_conv_desc& d);
int launch_direct_tc2t(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                       cudaStream_t st, bool y_nchw = false);
// d: an NHWC descriptor.  True if the kernel chosen for it can store its result NCHW itself (launch_direct_tc with y_nchw).
bool direct_tc_stores_nchw(const wino_conv_desc& d);

}  // namespace wino

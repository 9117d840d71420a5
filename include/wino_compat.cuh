// wino_compat.cuh — the reference's convolution entry points, same names and signatures, forwarding to libwino.
//
// Include this where the reference includes "DataLayoutTrans.cuh" / "wrapedConv_<L>.cuh"
// (comparison/layoutCompare.cu:8-11, netTest/cudnn_test_0124/VGG_Batched/Network.h) and link with -lwino: a
// layoutCompare.cu-shaped host then compiles unchanged.  Semantics kept from the reference: FP32 arithmetic,
// F(4x4,3x3), square images, caller-owned device workspaces of the reference's minimum sizes, `chn` updated
// to numOfFilter, device synchronised on return, *output written in place.  The reference wrappers return void
// and ignore errors; these print libwino's message to stderr.
#pragma once

#include <cstdio>

#include "wino.h"

#ifndef WARMUP
#define WARMUP
__global__ void warmup() {}                    // comparison/wrapedConv_NCHW.cuh:6
#endif

enum class DataLayout { NCHW, NHWC, CHWN };    // comparison/DataLayoutTrans.cuh:587-591 (same order as WINO_*)

// comparison/DataLayoutTrans.cuh:594-651
inline void layoutManager(DataLayout srcLayout, DataLayout dstLayout, int bat4Conv, int inside, int& chn, int numOfFilter,
                          int padding, float* input, float* weights, float* inputTran_gpu, float* filterTran_gpu,
                          float* gemmOutput_gpu, float** output) {
    if (wino_wraped_conv((int)srcLayout, (int)dstLayout, bat4Conv, inside, &chn, numOfFilter, padding, input, weights,
                         inputTran_gpu, filterTran_gpu, gemmOutput_gpu, output) != WINO_OK)
        fprintf(stderr, "libwino: %s\n", wino_last_error_string());
}

// comparison/wrapedConv_NCHW.cuh:8, wrapedConv_NHWC.cuh:8, wrapedConv_CHWN.cuh:8
#define WINO_COMPAT_SAME(L)                                                                                        \
    inline void wrapedConv_##L(int bat4Conv, int inside, int& chn, int numOfFilter, int padding, float* m1, float* m2, \
                               float* inputTran_gpu, float* filterTran_gpu, float* gemmOutput_gpu, float** output) {  \
        layoutManager(DataLayout::L, DataLayout::L, bat4Conv, inside, chn, numOfFilter, padding, m1, m2,           \
                      inputTran_gpu, filterTran_gpu, gemmOutput_gpu, output);                                       \
    }
WINO_COMPAT_SAME(NCHW)
WINO_COMPAT_SAME(NHWC)
WINO_COMPAT_SAME(CHWN)
#undef WINO_COMPAT_SAME

// comparison/DataLayoutTrans.cuh:9, 101, 192, 309, 418, 502
#define WINO_COMPAT_CROSS(S, D)                                                                                     \
    inline void convLayoutTrans_##S##_to_##D(int bat4Conv, int inside, int& chn, int numOfFilter, int padding,      \
                                             float* m1, float* m2, float* inputTran_gpu, float* filterTran_gpu,     \
                                             float* gemmOutput_gpu, float** output) {                               \
        layoutManager(DataLayout::S, DataLayout::D, bat4Conv, inside, chn, numOfFilter, padding, m1, m2,           \
                      inputTran_gpu, filterTran_gpu, gemmOutput_gpu, output);                                       \
    }
WINO_COMPAT_CROSS(CHWN, NCHW)
WINO_COMPAT_CROSS(CHWN, NHWC)
WINO_COMPAT_CROSS(NHWC, NCHW)
WINO_COMPAT_CROSS(NHWC, CHWN)
WINO_COMPAT_CROSS(NCHW, NHWC)
WINO_COMPAT_CROSS(NCHW, CHWN)
#undef WINO_COMPAT_CROSS

// wino_cudnn_compat.cuh — the reference's cuDNN comparator entry point, same name and signature.
//
// Include this where the reference includes "wrapedConv_CuDNN.cuh" (comparison/layoutCompare.cu:12, called at :194)
// and link with -lcudnn.  wrapedConv_CuDNN keeps the reference's signature, return type (void) and mode numbering
// (comparison/wrapedConv_CuDNN.cuh:10-81: mode 3 / 4 = NCHW with WINOGRAD_NONFUSED / WINOGRAD, 5 / 6 = the same two
// algorithms in NHWC; FP32 tensors, CUDNN_FMA_MATH), written against cuDNN 9.  Differences by design:
//   * the cuDNN workspace is kept between calls and grows on demand, so a timed call does not contain
//     cudaMalloc / cudaFree (the reference allocates and frees it inside the timed call, wrapedConv_CuDNN.cuh:51-79);
//   * failures are reported on stdout and leave *output and chn untouched (the reference aborts through NVIDIA's
//     sample macros); wino_cudnn_conv is the same call returning the cuDNN status for hosts that want it.
// This header has no dependency on libwino: it is the comparator, not the product.
#pragma once

#include <cuda_runtime.h>
#include <cudnn.h>

#include <cstdio>

#ifndef WARMUP
#define WARMUP
__global__ void warmup() {}                    // comparison/wrapedConv_CuDNN.cuh:5-8
#endif

// grow-only device buffer for cuDNN's workspace, one per process
inline void* wino_cudnn_workspace(size_t need) {
    static void* ptr = nullptr;
    static size_t bytes = 0;
    if (need > bytes) {
        if (ptr) cudaFree(ptr);
        ptr = nullptr;
        bytes = 0;
        if (cudaMalloc(&ptr, need) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        bytes = need;
    }
    return ptr;
}

// Returns the cuDNN status as an int (0 = success, -1 = bad mode or no workspace memory).
inline int wino_cudnn_conv(int bat4Conv, int inside, int& chn, int numOfFilter, int padding, float* m1, float* m2,
                           float** output, int mode, cudnnHandle_t& handle, cudnnTensorDescriptor_t& xdesc,
                           cudnnTensorDescriptor_t& ydesc, cudnnFilterDescriptor_t& wdesc,
                           cudnnConvolutionDescriptor_t& conv_desc) {
    if (mode < 3 || mode > 6) {
        printf("The mode is not right\n");     // comparison/wrapedConv_CuDNN.cuh:44-46
        return -1;
    }
    const cudnnTensorFormat_t fmt = (mode == 3 || mode == 4) ? CUDNN_TENSOR_NCHW : CUDNN_TENSOR_NHWC;
    const cudnnConvolutionFwdAlgo_t algo =
        (mode == 3 || mode == 5) ? CUDNN_CONVOLUTION_FWD_ALGO_WINOGRAD_NONFUSED : CUDNN_CONVOLUTION_FWD_ALGO_WINOGRAD;
    const char* algo_name = (mode == 3 || mode == 5) ? "WINOGRAD_NONFUSED" : "WINOGRAD";
    const int oside = inside + 2 * padding - 2;
    cudnnStatus_t st;
#define WINO_CUDNN_TRY(expr)                                                                     \
    if ((st = (expr)) != CUDNN_STATUS_SUCCESS) {                                                 \
        printf("cuDNN: %s failed: %s\n", #expr, cudnnGetErrorString(st));                        \
        return (int)st;                                                                          \
    }
    WINO_CUDNN_TRY(cudnnSetTensor4dDescriptor(xdesc, fmt, CUDNN_DATA_FLOAT, bat4Conv, chn, inside, inside));
    WINO_CUDNN_TRY(cudnnSetTensor4dDescriptor(ydesc, fmt, CUDNN_DATA_FLOAT, bat4Conv, numOfFilter, oside, oside));
    WINO_CUDNN_TRY(cudnnSetFilter4dDescriptor(wdesc, CUDNN_DATA_FLOAT, fmt, numOfFilter, chn, 3, 3));
    WINO_CUDNN_TRY(cudnnSetConvolution2dDescriptor(conv_desc, padding, padding, 1, 1, 1, 1, CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT));
    WINO_CUDNN_TRY(cudnnSetConvolutionMathType(conv_desc, CUDNN_FMA_MATH));
#undef WINO_CUDNN_TRY
    size_t ws = 0;
    st = cudnnGetConvolutionForwardWorkspaceSize(handle, xdesc, wdesc, conv_desc, ydesc, algo, &ws);
    if (st != CUDNN_STATUS_SUCCESS) {
        printf("cuDNN %s not available for this shape: %s\n", algo_name, cudnnGetErrorString(st));
        return (int)st;
    }
    void* extra = wino_cudnn_workspace(ws ? ws : 16);
    if (!extra) {
        printf("cuDNN %s: no device memory for a workspace of %zu bytes\n", algo_name, ws);
        return -1;
    }
    const float one = 1.f, zero = 0.f;
    st = cudnnConvolutionForward(handle, &one, xdesc, m1, wdesc, m2, conv_desc, algo, extra, ws, &zero, ydesc, *output);
    if (st != CUDNN_STATUS_SUCCESS) {
        printf("cuDNN %s failed: %s\n", algo_name, cudnnGetErrorString(st));
        return (int)st;
    }
    chn = numOfFilter;                         // comparison/wrapedConv_CuDNN.cuh:80
    return 0;
}

// comparison/wrapedConv_CuDNN.cuh:10
inline void wrapedConv_CuDNN(int bat4Conv, int inside, int& chn, int numOfFilter, int padding, float* m1, float* m2,
                             float** output, int mode, cudnnHandle_t& handle, cudnnTensorDescriptor_t& xdesc,
                             cudnnTensorDescriptor_t& ydesc, cudnnFilterDescriptor_t& wdesc,
                             cudnnConvolutionDescriptor_t& conv_desc) {
    (void)wino_cudnn_conv(bat4Conv, inside, chn, numOfFilter, padding, m1, m2, output, mode, handle, xdesc, ydesc, wdesc, conv_desc);
}

// cuDNN comparator of the harnesses.
//
// wrapedConv_CuDNN with the reference's signature (comparison/wrapedConv_CuDNN.cuh:10-81) lives in
// include/wino_cudnn_compat.cuh, next to the other drop-in headers; wino_cudnn_conv there returns the status.
// cudnn_best_forward times every algorithm cudnnFindConvolutionForwardAlgorithm reports as working for a given
// tensor format, data type and math mode and returns the fastest: the "cuDNN best" baseline.
#pragma once

#include <cudnn.h>

#include <string>

#include "harness_common.h"
#include "wino_cudnn_compat.cuh"

#define HCHECK_CUDNN(expr)                                                                               \
    do {                                                                                                 \
        cudnnStatus_t s_ = (expr);                                                                       \
        if (s_ != CUDNN_STATUS_SUCCESS) {                                                                \
            fprintf(stderr, "%s:%d: %s failed: %s\n", __FILE__, __LINE__, #expr, cudnnGetErrorString(s_)); \
            exit(4);                                                                                     \
        }                                                                                                \
    } while (0)

namespace harness {

inline const char* fwd_algo_name(int a) {
    static const char* n[] = {"IMPLICIT_GEMM", "IMPLICIT_PRECOMP_GEMM", "GEMM", "DIRECT", "FFT", "FFT_TILING", "WINOGRAD",
                              "WINOGRAD_NONFUSED"};
    return a >= 0 && a < 8 ? n[a] : "?";
}

struct CudnnWorkspace {
    void* ptr = nullptr;
    size_t bytes = 0;
    void* reserve(size_t need) {
        if (need > bytes) {
            if (ptr) cudaFree(ptr);
            HCHECK_CUDA(cudaMalloc(&ptr, need));
            bytes = need;
        }
        return ptr;
    }
};
inline CudnnWorkspace& cudnn_workspace() {
    static CudnnWorkspace w;
    return w;
}

struct CudnnBest {
    double ms = -1;
    int algo = -1;
    std::string tried;
};

// dtype: WINO_FP32 (CUDNN_FMA_MATH, exact), WINO_TF32 (float data, tensor-op math allowed), WINO_BF16 (bf16 data).
// x, w, y are device buffers in `fmt` (filters in the same format: KCRS for NCHW, KRSC for NHWC).
inline CudnnBest cudnn_best_forward(cudnnHandle_t handle, cudnnTensorFormat_t fmt, int dtype, int n, int c, int h, int w,
                                    int k, int pad, const void* x, const void* wt, void* y, int warm = 5, int iters = 20) {
    cudnnTensorDescriptor_t xd, yd;
    cudnnFilterDescriptor_t wd;
    cudnnConvolutionDescriptor_t cd;
    HCHECK_CUDNN(cudnnCreateTensorDescriptor(&xd));
    HCHECK_CUDNN(cudnnCreateTensorDescriptor(&yd));
    HCHECK_CUDNN(cudnnCreateFilterDescriptor(&wd));
    HCHECK_CUDNN(cudnnCreateConvolutionDescriptor(&cd));
    const cudnnDataType_t dt = dtype == WINO_BF16 ? CUDNN_DATA_BFLOAT16 : CUDNN_DATA_FLOAT;
    const int oh = h + 2 * pad - 2, ow = w + 2 * pad - 2;
    HCHECK_CUDNN(cudnnSetTensor4dDescriptor(xd, fmt, dt, n, c, h, w));
    HCHECK_CUDNN(cudnnSetTensor4dDescriptor(yd, fmt, dt, n, k, oh, ow));
    HCHECK_CUDNN(cudnnSetFilter4dDescriptor(wd, dt, fmt, k, c, 3, 3));
    HCHECK_CUDNN(cudnnSetConvolution2dDescriptor(cd, pad, pad, 1, 1, 1, 1, CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT));
    HCHECK_CUDNN(cudnnSetConvolutionMathType(cd, dtype == WINO_FP32 ? CUDNN_FMA_MATH : CUDNN_TENSOR_OP_MATH_ALLOW_CONVERSION));
    CudnnBest best;
    cudaEvent_t e0, e1;
    HCHECK_CUDA(cudaEventCreate(&e0));
    HCHECK_CUDA(cudaEventCreate(&e1));
    const float one = 1.f, zero = 0.f;
    for (int a = 0; a < 8; ++a) {
        const cudnnConvolutionFwdAlgo_t algo = (cudnnConvolutionFwdAlgo_t)a;
        size_t ws = 0;
        if (cudnnGetConvolutionForwardWorkspaceSize(handle, xd, wd, cd, yd, algo, &ws) != CUDNN_STATUS_SUCCESS) {
            best.tried += std::string(fwd_algo_name(a)) + ":unsupported ";
            continue;
        }
        if (ws > (size_t)16 << 30) {
            best.tried += std::string(fwd_algo_name(a)) + ":workspace>16GiB ";
            continue;
        }
        void* extra = cudnn_workspace().reserve(ws ? ws : 16);
        bool ok = true;
        for (int i = 0; i < warm && ok; ++i)
            ok = cudnnConvolutionForward(handle, &one, xd, x, wd, wt, cd, algo, extra, ws, &zero, yd, y) == CUDNN_STATUS_SUCCESS;
        if (!ok || cudaDeviceSynchronize() != cudaSuccess) {
            cudaGetLastError();
            best.tried += std::string(fwd_algo_name(a)) + ":failed ";
            continue;
        }
        HCHECK_CUDA(cudaEventRecord(e0));
        for (int i = 0; i < iters; ++i) cudnnConvolutionForward(handle, &one, xd, x, wd, wt, cd, algo, extra, ws, &zero, yd, y);
        HCHECK_CUDA(cudaEventRecord(e1));
        HCHECK_CUDA(cudaEventSynchronize(e1));
        float ms = 0;
        HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        ms /= iters;
        char buf[64];
        snprintf(buf, sizeof(buf), "%s:%.3fms ", fwd_algo_name(a), ms);
        best.tried += buf;
        if (best.ms < 0 || ms < best.ms) { best.ms = ms; best.algo = a; }
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudnnDestroyTensorDescriptor(xd);
    cudnnDestroyTensorDescriptor(yd);
    cudnnDestroyFilterDescriptor(wd);
    cudnnDestroyConvolutionDescriptor(cd);
    return best;
}

}  // namespace harness

// The classifier tail of the reference's VGG-16 harness: fc14 (25088 -> 4096) + ReLU, fc15 (4096 -> 4096) + ReLU,
// fc16 (4096 -> 1000), softmax, arg-max per image
// (netTest/cudnn_test_0124/VGG_Batched/Network.h:145-169 fullyConnectedForward = bias copy + cuBLAS gemm,
//  :368-386 softmaxForward = cudnnSoftmaxForward ACCURATE / MODE_CHANNEL, :668-704 the call sequence and the arg-max;
//  weights "vggData/fc14.bin", "fc14.bias.bin", ... as float32, [outputs][inputs], vggCUDNN.cu:39-44, :178-180).
// It sits outside the convolution hot path: the three products are plain library GEMMs (cuBLAS, FP32), the bias /
// ReLU / softmax / flatten steps are small kernels here.  The reference's arg-max keeps its running index across
// images (Network.h:690-700, `id` is never reset); here every image starts from class 0.
#pragma once

#include <cublas_v2.h>

#include "harness_common.h"

namespace harness {

#define HCHECK_CUBLAS(expr)                                                                     \
    do {                                                                                        \
        cublasStatus_t s_ = (expr);                                                             \
        if (s_ != CUBLAS_STATUS_SUCCESS) {                                                      \
            fprintf(stderr, "cuBLAS error %d at %s:%d\n", (int)s_, __FILE__, __LINE__);         \
            exit(4);                                                                            \
        }                                                                                       \
    } while (0)

__global__ void tail_bf16_to_float(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, long long count) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = __bfloat162float(in[i]);
}

// y[n][o] += b[o], optional ReLU
__global__ void tail_bias_act(float* __restrict__ y, const float* __restrict__ b, int outputs, long long count, int relu) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float v = y[i] + b[i % outputs];
    y[i] = relu ? fmaxf(v, 0.f) : v;
}

// one block per image: p = exp(x - max) / sum (the "accurate" softmax), and the arg-max
__global__ void tail_softmax_argmax(const float* __restrict__ logits, float* __restrict__ prob, int* __restrict__ top1, int classes) {
    __shared__ float red[256];
    __shared__ int redi[256];
    const float* x = logits + (long long)blockIdx.x * classes;
    float* p = prob + (long long)blockIdx.x * classes;
    float mx = -INFINITY;
    int mi = 0;
    for (int i = threadIdx.x; i < classes; i += blockDim.x)
        if (x[i] > mx) { mx = x[i]; mi = i; }
    red[threadIdx.x] = mx; redi[threadIdx.x] = mi;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float o = red[threadIdx.x + s];
            const int oi = redi[threadIdx.x + s];
            if (o > red[threadIdx.x] || (o == red[threadIdx.x] && oi < redi[threadIdx.x])) { red[threadIdx.x] = o; redi[threadIdx.x] = oi; }
        }
        __syncthreads();
    }
    mx = red[0];
    if (threadIdx.x == 0) top1[blockIdx.x] = redi[0];
    __syncthreads();
    float sum = 0.f;
    for (int i = threadIdx.x; i < classes; i += blockDim.x) sum += expf(x[i] - mx);
    red[threadIdx.x] = sum;
    __syncthreads();
    for (int s = blockDim.x / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) red[threadIdx.x] += red[threadIdx.x + s];
        __syncthreads();
    }
    sum = red[0];
    for (int i = threadIdx.x; i < classes; i += blockDim.x) p[i] = expf(x[i] - mx) / sum;
}

struct ClassifierTail {
    static constexpr int kIn[3] = {25088, 4096, 4096};
    static constexpr int kOut[3] = {4096, 4096, 1000};
    int n = 0;
    bool from_files = true;
    cublasHandle_t handle = nullptr;
    std::vector<float> w_h[3], b_h[3];
    float *w_d[3] = {}, *b_d[3] = {};
    float *flat = nullptr, *a14 = nullptr, *a15 = nullptr, *logits = nullptr, *prob = nullptr;
    void* nchw = nullptr;       // the last convolution output relaid out to NCHW (storage dtype)
    int* top1_d = nullptr;

    void init(int batch) {
        n = batch;
        HCHECK_CUBLAS(cublasCreate(&handle));
        static const char* wn[3] = {"./vggData/fc14.bin", "./vggData/fc15.bin", "./vggData/fc16.bin"};
        static const char* bn[3] = {"./vggData/fc14.bias.bin", "./vggData/fc15.bias.bin", "./vggData/fc16.bias.bin"};
        for (int l = 0; l < 3; ++l) {
            w_h[l].resize((size_t)kIn[l] * kOut[l]);
            b_h[l].resize(kOut[l]);
            if (!read_floats(wn[l], w_h[l].data(), w_h[l].size()) || !read_floats(bn[l], b_h[l].data(), b_h[l].size())) {
                from_files = false;     // the pretrained weights are not shipped: seeded He-normal stand-ins
                fill_normal(w_h[l].data(), w_h[l].size(), 300 + l, std::sqrt(2.f / kIn[l]));
                fill_normal(b_h[l].data(), b_h[l].size(), 400 + l, 0.01f);
            }
            HCHECK_CUDA(cudaMalloc(&w_d[l], w_h[l].size() * 4));
            HCHECK_CUDA(cudaMalloc(&b_d[l], b_h[l].size() * 4));
            HCHECK_CUDA(cudaMemcpy(w_d[l], w_h[l].data(), w_h[l].size() * 4, cudaMemcpyHostToDevice));
            HCHECK_CUDA(cudaMemcpy(b_d[l], b_h[l].data(), b_h[l].size() * 4, cudaMemcpyHostToDevice));
        }
        HCHECK_CUDA(cudaMalloc(&flat, (size_t)n * kIn[0] * 4));
        HCHECK_CUDA(cudaMalloc(&nchw, (size_t)n * kIn[0] * 4));
        HCHECK_CUDA(cudaMalloc(&a14, (size_t)n * kOut[0] * 4));
        HCHECK_CUDA(cudaMalloc(&a15, (size_t)n * kOut[1] * 4));
        HCHECK_CUDA(cudaMalloc(&logits, (size_t)n * kOut[2] * 4));
        HCHECK_CUDA(cudaMalloc(&prob, (size_t)n * kOut[2] * 4));
        HCHECK_CUDA(cudaMalloc(&top1_d, n * sizeof(int)));
    }

    // y[n][out] = x[n][in] . W[out][in]^T (+ bias, optional ReLU)
    void fc(int l, const float* x, float* y, bool relu) {
        const float one = 1.f, zero = 0.f;
        HCHECK_CUBLAS(cublasSgemm(handle, CUBLAS_OP_T, CUBLAS_OP_N, kOut[l], n, kIn[l], &one, w_d[l], kIn[l], x, kIn[l], &zero, y, kOut[l]));
        const long long count = (long long)n * kOut[l];
        tail_bias_act<<<(unsigned)((count + 255) / 256), 256>>>(y, b_d[l], kOut[l], count, relu ? 1 : 0);
    }

    // conv_out: the pooled output of conv13, (n, 512, 7, 7) in `layout`, storage `dtype`
    void forward(const void* conv_out, int layout, int dtype) {
        const void* src = conv_out;
        if (layout != WINO_NCHW) {      // the reference flattens NCHW data: index c*49 + h*7 + w
            HCHECK_WINO(wino_layout_convert(layout, WINO_NCHW, n, 512, 7, 7, dtype, conv_out, nchw, nullptr));
            src = nchw;
        }
        const long long count = (long long)n * kIn[0];
        if (dtype == WINO_BF16)
            tail_bf16_to_float<<<(unsigned)((count + 255) / 256), 256>>>((const __nv_bfloat16*)src, flat, count);
        else
            HCHECK_CUDA(cudaMemcpyAsync(flat, src, count * 4, cudaMemcpyDeviceToDevice, nullptr));
        fc(0, flat, a14, true);
        fc(1, a14, a15, true);
        fc(2, a15, logits, false);
        tail_softmax_argmax<<<n, 256>>>(logits, prob, top1_d, kOut[2]);
        HCHECK_CUDA(cudaGetLastError());
    }

    // Host restatement (double accumulation) of the tail for one image from the device's flattened input; returns the
    // largest |p - p_ref| over the 1000 classes and whether the arg-max agrees.
    double check_image(int img, bool* top1_ok) {
        std::vector<float> x(kIn[0]), p(kOut[2]);
        HCHECK_CUDA(cudaMemcpy(x.data(), flat + (size_t)img * kIn[0], x.size() * 4, cudaMemcpyDeviceToHost));
        HCHECK_CUDA(cudaMemcpy(p.data(), prob + (size_t)img * kOut[2], p.size() * 4, cudaMemcpyDeviceToHost));
        int dev_top1 = 0;
        HCHECK_CUDA(cudaMemcpy(&dev_top1, top1_d + img, sizeof(int), cudaMemcpyDeviceToHost));
        std::vector<double> cur(x.begin(), x.end()), next;
        for (int l = 0; l < 3; ++l) {
            next.assign(kOut[l], 0.0);
            for (int o = 0; o < kOut[l]; ++o) {
                double acc = b_h[l][o];
                const float* wr = w_h[l].data() + (size_t)o * kIn[l];
                for (int i = 0; i < kIn[l]; ++i) acc += cur[i] * (double)wr[i];
                next[o] = (l < 2 && acc < 0) ? 0.0 : acc;
            }
            cur.swap(next);
        }
        double mx = cur[0];
        int arg = 0;
        for (int i = 1; i < kOut[2]; ++i)
            if (cur[i] > mx) { mx = cur[i]; arg = i; }
        double sum = 0;
        for (double v : cur) sum += std::exp(v - mx);
        double worst = 0;
        for (int i = 0; i < kOut[2]; ++i) worst = std::fmax(worst, std::fabs(std::exp(cur[i] - mx) / sum - (double)p[i]));
        *top1_ok = arg == dev_top1;
        return worst;
    }

    std::vector<int> top1() {
        std::vector<int> t(n);
        HCHECK_CUDA(cudaMemcpy(t.data(), top1_d, n * sizeof(int), cudaMemcpyDeviceToHost));
        return t;
    }
};

}  // namespace harness

// netTest — VGG-16 convolution stack, this library against cuDNN, whole-network timing.
//
// Takes the role of the convolutional part of netTest/cudnn_test_0124/VGG_Batched (main vggCUDNN.cu:72-298,
// classify_example_modified Network.h:521-706, timed region :594-679): 13 3x3 pad-1 convolutions with bias and
// ReLU, a 2x2 max-pool after each of the five blocks.  Command line as there: `netTest set batch=B mode=M`
//   mode 0/1/2   this library in NCHW / NHWC / CHWN: one wino_conv_forward per layer (bias, ReLU and the pool
//                fused into the output transform) instead of the reference's 6-7 kernels per layer
//                (layoutManager + addBias + relu (+ pool), Network.h:456-519, :603-669).  In mode 2 the last
//                convolution reads CHWN and writes NCHW, the hand-off to the classifier that the reference makes
//                at conv13 (vggCUDNN.cu:173-176); with tail=1 it also writes FP32 whatever the storage type of the
//                stack, so the classifier's FP32 GEMM reads it without a relayout or conversion pass
//   mode 3/4     cuDNN in NCHW / NHWC: fastest forward algorithm per layer + cudnnAddTensor +
//                cudnnActivationForward (+ cudnnPoolingForward), i.e. Network.h:171-312, :314-444
// plus dtype=fp32|fp32x3|tf32|bf16 (default bf16), rounds= (default 10), tail=0|1, fusepool=1|0 (0: modes 0-2 run the
// block-end pooling as its own pass, wino_maxpool2x2, the way the reference sequences it, Network.h:314-366, :603-669).  With tail=1 the classifier tail of the
// reference (fc14 + ReLU, fc15 + ReLU, fc16, softmax, arg-max: Network.h:668-704) runs after the last round on the
// output of conv13 (classifier_tail.h: cuBLAS GEMMs + small kernels), is checked against a host restatement for two
// images and reports the top-1 classes.  The pretrained weights (./vggData/*.bin) and ImageNet batches the reference
// reads are not shipped; they are used if present, otherwise weights are seeded He-normal and the input
// uniform[-1,1] (so the classes mean nothing, the arithmetic is what is checked).  Prints "time:<ms> ms" per round
// and a JSON summary.
#include "classifier_tail.h"
#include "cudnn_compare.h"
#include "harness_common.h"

using namespace harness;

struct Layer { int c, k, s; bool pool; };
static const Layer kVgg[13] = {{3, 64, 224, false},  {64, 64, 224, true},   {64, 128, 112, false}, {128, 128, 112, true},
                               {128, 256, 56, false}, {256, 256, 56, false}, {256, 256, 56, true},  {256, 512, 28, false},
                               {512, 512, 28, false}, {512, 512, 28, true},  {512, 512, 14, false}, {512, 512, 14, false},
                               {512, 512, 14, true}};

int main(int argc, char** argv) {
    const int n = (int)arg_int(argc, argv, "batch", 32);
    const int mode = (int)arg_int(argc, argv, "mode", 1);
    const int rounds = (int)arg_int(argc, argv, "rounds", 10);
    const int tail = (int)arg_int(argc, argv, "tail", 0);
    const int fusepool = (int)arg_int(argc, argv, "fusepool", 1);
    const std::string dts = arg_str(argc, argv, "dtype", "bf16");
    const int dtype = dts == "bf16" ? WINO_BF16 : dts == "tf32" ? WINO_TF32 : dts == "fp32x3" ? WINO_FP32X3 : WINO_FP32;
    const int cudnn_dtype = dtype == WINO_FP32X3 ? WINO_FP32 : dtype;   // FP32-accurate variants face cuDNN's CUDNN_FMA_MATH
    HCHECK_CUDA(cudaSetDevice((int)arg_int(argc, argv, "device", 0)));
    if (mode < 0 || mode > 4 || n <= 0) { fprintf(stderr, "mode must be 0..4, batch positive\n"); return 1; }
    const int layout = mode <= 2 ? mode : mode == 3 ? WINO_NCHW : WINO_NHWC;
    const size_t es = dtype == WINO_BF16 ? 2 : 4;

    // activations ping-pong between two buffers sized for the largest tensor (224*224*64 per image)
    const size_t max_act = (size_t)n * 64 * 224 * 224;
    void* act[2];
    HCHECK_CUDA(cudaMalloc(&act[0], max_act * es));
    HCHECK_CUDA(cudaMalloc(&act[1], max_act * es));
    void* input;
    {
        std::vector<float> x((size_t)n * 3 * 224 * 224);
        fill_uniform(x.data(), x.size(), 1, -1.f, 1.f);
        x = to_layout(x, layout, n, 3, 224, 224);
        HCHECK_CUDA(cudaMalloc(&input, x.size() * es));
        if (dtype == WINO_BF16) {
            auto xb = to_bf16(x);
            HCHECK_CUDA(cudaMemcpy(input, xb.data(), x.size() * 2, cudaMemcpyHostToDevice));
        } else {
            HCHECK_CUDA(cudaMemcpy(input, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
        }
    }
    std::vector<void*> wdev(13), bdev(13);
    for (int l = 0; l < 13; ++l) {
        const Layer& L = kVgg[l];
        std::vector<float> w((size_t)9 * L.k * L.c), b(L.k);
        fill_normal(w.data(), w.size(), 100 + l, std::sqrt(2.f / (9.f * L.c)));
        fill_normal(b.data(), b.size(), 200 + l, 0.01f);
        w = filter_to_layout(w, layout, L.k, L.c);
        HCHECK_CUDA(cudaMalloc(&wdev[l], w.size() * es));
        if (dtype == WINO_BF16) {
            auto wb = to_bf16(w);
            HCHECK_CUDA(cudaMemcpy(wdev[l], wb.data(), w.size() * 2, cudaMemcpyHostToDevice));
        } else {
            HCHECK_CUDA(cudaMemcpy(wdev[l], w.data(), w.size() * 4, cudaMemcpyHostToDevice));
        }
        HCHECK_CUDA(cudaMalloc(&bdev[l], L.k * 4));
        HCHECK_CUDA(cudaMemcpy(bdev[l], b.data(), L.k * 4, cudaMemcpyHostToDevice));
    }

    cudaEvent_t e0, e1;
    HCHECK_CUDA(cudaEventCreate(&e0));
    HCHECK_CUDA(cudaEventCreate(&e1));
    std::vector<float> times;
    std::string what;
    const void* final_out = nullptr;      // pooled output of conv13: (n, 512, 7, 7) in `final_layout`, stored as `final_dtype`
    int final_layout = layout, final_dtype = dtype;

    if (mode <= 2) {
        std::vector<wino_conv_desc> desc(13);
        std::vector<void*> u(13);
        size_t wsb = 0;
        for (int l = 0; l < 13; ++l) {
            wino_conv_desc& d = desc[l];
            memset(&d, 0, sizeof(d));
            d.layout_in = d.layout_out = layout;
            d.n = n; d.c = kVgg[l].c; d.h = d.w = kVgg[l].s; d.k = kVgg[l].k; d.pad = 1;
            d.dtype = dtype; d.relu = 1; d.has_bias = 1; d.pool2x2 = kVgg[l].pool && fusepool;
            if (mode == 2 && l == 12) {        // conv13.layout_in = CHWN, layout_out = NCHW (vggCUDNN.cu:173-176)
                d.layout_out = final_layout = WINO_NCHW;
                if (tail) { d.out_dtype = WINO_OUT_FP32; final_dtype = dtype == WINO_BF16 ? WINO_FP32 : dtype; }
            }
            const size_t ub = wino_filter_bytes(&d), wb = wino_conv_workspace_bytes(&d);
            if (!ub || !wb) { fprintf(stderr, "libwino: %s\n", wino_last_error_string()); return 3; }
            HCHECK_CUDA(cudaMalloc(&u[l], ub));
            HCHECK_WINO(wino_filter_transform(&d, wdev[l], u[l], nullptr));   // once per weight tensor
            wsb = wb > wsb ? wb : wsb;
        }
        void* ws;
        HCHECK_CUDA(cudaMalloc(&ws, wsb));
        for (int r = 0; r < rounds + 2; ++r) {
            HCHECK_CUDA(cudaEventRecord(e0));
            const void* cur = input;
            int slot = 0;
            for (int l = 0; l < 13; ++l) {
                void* out = act[slot];
                HCHECK_WINO(wino_conv_forward(&desc[l], cur, u[l], (const float*)bdev[l], out, ws, wsb, nullptr));
                cur = out;
                slot ^= 1;
                if (kVgg[l].pool && !fusepool) {     // the pooling pass on its own, in the layout and type the layer wrote
                    const int pdt = desc[l].out_dtype == WINO_OUT_FP32 ? WINO_FP32 : dtype;
                    HCHECK_WINO(wino_maxpool2x2(desc[l].layout_out, n, kVgg[l].k, kVgg[l].s, kVgg[l].s, pdt, cur, act[slot], nullptr));
                    cur = act[slot];
                    slot ^= 1;
                }
            }
            HCHECK_CUDA(cudaEventRecord(e1));
            HCHECK_CUDA(cudaEventSynchronize(e1));
            float ms;
            HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
            if (r >= 2) times.push_back(ms);
            final_out = cur;
        }
        HCHECK_WINO(wino_device_status());
        what = fusepool ? "libwino: one fused conv+bias+ReLU(+pool) call per layer" : "libwino: fused conv+bias+ReLU per layer, pooling as a separate pass";
    } else {
        cudnnHandle_t handle;
        HCHECK_CUDNN(cudnnCreate(&handle));
        const cudnnTensorFormat_t fmt = mode == 3 ? CUDNN_TENSOR_NCHW : CUDNN_TENSOR_NHWC;
        const cudnnDataType_t dt = dtype == WINO_BF16 ? CUDNN_DATA_BFLOAT16 : CUDNN_DATA_FLOAT;
        // pick the fastest algorithm per distinct layer shape first (outside the timed region)
        std::vector<int> algo(13, -1);
        for (int l = 0; l < 13; ++l) {
            for (int p = 0; p < l; ++p)
                if (kVgg[p].c == kVgg[l].c && kVgg[p].k == kVgg[l].k && kVgg[p].s == kVgg[l].s) algo[l] = algo[p];
            if (algo[l] < 0) {
                const CudnnBest b = cudnn_best_forward(handle, fmt, cudnn_dtype, n, kVgg[l].c, kVgg[l].s, kVgg[l].s, kVgg[l].k, 1,
                                                       l == 0 ? input : act[0], wdev[l], act[1], 2, 5);
                if (b.algo < 0) { printf("{\"harness\": \"netTest\", \"mode\": %d, \"unsupported\": \"layer %d: %s\"}\n", mode, l + 1, b.tried.c_str()); return 0; }
                algo[l] = b.algo;
            }
        }
        cudnnTensorDescriptor_t xd, yd, bd, pd;
        cudnnFilterDescriptor_t wd;
        cudnnConvolutionDescriptor_t cd;
        cudnnActivationDescriptor_t ad;
        cudnnPoolingDescriptor_t pool;
        HCHECK_CUDNN(cudnnCreateTensorDescriptor(&xd));
        HCHECK_CUDNN(cudnnCreateTensorDescriptor(&yd));
        HCHECK_CUDNN(cudnnCreateTensorDescriptor(&bd));
        HCHECK_CUDNN(cudnnCreateTensorDescriptor(&pd));
        HCHECK_CUDNN(cudnnCreateFilterDescriptor(&wd));
        HCHECK_CUDNN(cudnnCreateConvolutionDescriptor(&cd));
        HCHECK_CUDNN(cudnnCreateActivationDescriptor(&ad));
        HCHECK_CUDNN(cudnnCreatePoolingDescriptor(&pool));
        HCHECK_CUDNN(cudnnSetActivationDescriptor(ad, CUDNN_ACTIVATION_RELU, CUDNN_PROPAGATE_NAN, 0.0));
        HCHECK_CUDNN(cudnnSetPooling2dDescriptor(pool, CUDNN_POOLING_MAX, CUDNN_PROPAGATE_NAN, 2, 2, 0, 0, 2, 2));
        HCHECK_CUDNN(cudnnSetConvolution2dDescriptor(cd, 1, 1, 1, 1, 1, 1, CUDNN_CROSS_CORRELATION, CUDNN_DATA_FLOAT));
        HCHECK_CUDNN(cudnnSetConvolutionMathType(cd, cudnn_dtype == WINO_FP32 ? CUDNN_FMA_MATH : CUDNN_TENSOR_OP_MATH_ALLOW_CONVERSION));
        void* bias_t[13];   // biases in the tensor data type, as cudnnAddTensor wants
        for (int l = 0; l < 13; ++l) {
            bias_t[l] = bdev[l];
            if (dtype == WINO_BF16) {
                std::vector<float> b(kVgg[l].k);
                HCHECK_CUDA(cudaMemcpy(b.data(), bdev[l], b.size() * 4, cudaMemcpyDeviceToHost));
                auto bb = to_bf16(b);
                HCHECK_CUDA(cudaMalloc(&bias_t[l], bb.size() * 2));
                HCHECK_CUDA(cudaMemcpy(bias_t[l], bb.data(), bb.size() * 2, cudaMemcpyHostToDevice));
            }
        }
        const float one = 1.f, zero = 0.f;
        for (int r = 0; r < rounds + 2; ++r) {
            HCHECK_CUDA(cudaEventRecord(e0));
            const void* cur = input;
            int slot = 0;
            for (int l = 0; l < 13; ++l) {
                const Layer& L = kVgg[l];
                HCHECK_CUDNN(cudnnSetTensor4dDescriptor(xd, fmt, dt, n, L.c, L.s, L.s));
                HCHECK_CUDNN(cudnnSetTensor4dDescriptor(yd, fmt, dt, n, L.k, L.s, L.s));
                HCHECK_CUDNN(cudnnSetTensor4dDescriptor(bd, fmt, dt, 1, L.k, 1, 1));
                HCHECK_CUDNN(cudnnSetFilter4dDescriptor(wd, dt, fmt, L.k, L.c, 3, 3));
                size_t wsz = 0;
                HCHECK_CUDNN(cudnnGetConvolutionForwardWorkspaceSize(handle, xd, wd, cd, yd, (cudnnConvolutionFwdAlgo_t)algo[l], &wsz));
                void* extra = cudnn_workspace().reserve(wsz ? wsz : 16);
                void* out = act[slot];
                HCHECK_CUDNN(cudnnConvolutionForward(handle, &one, xd, cur, wd, wdev[l], cd, (cudnnConvolutionFwdAlgo_t)algo[l], extra, wsz, &zero, yd, out));
                HCHECK_CUDNN(cudnnAddTensor(handle, &one, bd, bias_t[l], &one, yd, out));
                HCHECK_CUDNN(cudnnActivationForward(handle, ad, &one, yd, out, &zero, yd, out));
                cur = out;
                slot ^= 1;
                if (L.pool) {
                    HCHECK_CUDNN(cudnnSetTensor4dDescriptor(pd, fmt, dt, n, L.k, L.s / 2, L.s / 2));
                    HCHECK_CUDNN(cudnnPoolingForward(handle, pool, &one, yd, cur, &zero, pd, act[slot]));
                    cur = act[slot];
                    slot ^= 1;
                }
            }
            HCHECK_CUDA(cudaEventRecord(e1));
            HCHECK_CUDA(cudaEventSynchronize(e1));
            float ms;
            HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
            if (r >= 2) times.push_back(ms);
            final_out = cur;
        }
        what = "cuDNN: fastest forward algorithm per layer + AddTensor + ActivationForward (+ PoolingForward)";
        cudnnDestroy(handle);
    }

    double sum = 0, best = 1e30;
    for (float t : times) {
        printf("time:%lf ms\n", (double)t);
        sum += t;
        best = t < best ? t : best;
    }
    const double avg = sum / times.size();
    double flops = 0;
    for (const Layer& L : kVgg) flops += 2.0 * L.k * L.c * (double)L.s * L.s * 9;
    std::string tail_json;
    if (tail && final_out) {
        ClassifierTail ct;
        ct.init(n);
        ct.forward(final_out, final_layout, final_dtype);          // warm-up (cuBLAS set-up)
        HCHECK_CUDA(cudaDeviceSynchronize());
        HCHECK_CUDA(cudaEventRecord(e0));
        ct.forward(final_out, final_layout, final_dtype);
        HCHECK_CUDA(cudaEventRecord(e1));
        HCHECK_CUDA(cudaEventSynchronize(e1));
        float tail_ms;
        HCHECK_CUDA(cudaEventElapsedTime(&tail_ms, e0, e1));
        bool ok0 = false, ok1 = false;
        const double err0 = ct.check_image(0, &ok0), err1 = ct.check_image(n - 1, &ok1);
        const std::vector<int> top1 = ct.top1();
        for (int i = 0; i < n && i < 8; ++i) printf("Batch %d Resulting weights from Softmax:%d\n", i, top1[i]);
        char buf[512];
        snprintf(buf, sizeof(buf), ", \"tail_ms\": %.4f, \"tail_weights\": \"%s\", \"tail_max_abs_err\": %.3e, \"tail_top1_agree\": %s, \"top1_first\": %d",
                 tail_ms, ct.from_files ? "vggData/*.bin" : "seeded", err0 > err1 ? err0 : err1, (ok0 && ok1) ? "true" : "false", top1[0]);
        tail_json = buf;
        if (!(err0 <= 1e-4 && err1 <= 1e-4)) printf("classifier tail error\n");
    }
    printf("{\"harness\": \"netTest\", \"mode\": %d, \"batch\": %d, \"layout\": \"%s\", \"dtype\": \"%s\", \"ms_avg\": %.4f, \"ms_min\": %.4f, "
           "\"images_per_s\": %.1f, \"tflops_direct_equiv\": %.2f, \"what\": \"%s\"%s}\n",
           mode, n, layout_name(layout), dts.c_str(), avg, best, n / (avg * 1e-3), flops * n / avg / 1e9, what.c_str(), tail_json.c_str());
    return 0;
}

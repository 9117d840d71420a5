// layoutCompare — per-layer benchmark: this library in the three layouts against cuDNN.
//
// Same command line and output as the reference's harness (comparison/layoutCompare.cu:27-232, driven by
// comparison/test.sh): `layoutCompare batch=B opt=O layer=L` runs 20 timed convolutions of VGG-16 layer L
// (1..9, comparison/layoutCompare.cu:41-82) and prints one "time:<ms> ms" line per run.
//   opt 0/1/2  this library, NCHW / NHWC / CHWN
//   opt 3..6   cuDNN WINOGRAD_NONFUSED / WINOGRAD in NCHW, then in NHWC (FP32, FMA math), as in the reference
//   opt 7/8    cuDNN's fastest forward algorithm in NCHW / NHWC for the chosen dtype ("cuDNN best")
// Additions: dtype=fp32|fp32x3|tf32|bf16 (default fp32, the reference's arithmetic; fp32x3 = split-TF32 tensor-core GEMM), wino=4|2|0 (0 = the engine's choice of
// kernel per layer, the default for tf32 / bf16; 4 = F(4x4,3x3) Winograd, the default for fp32), seed=, check=0|1,
// iters=.  With dtype=fp32 and opt 0..2 the timed call is layoutManager() through include/wino_compat.cuh, i.e.
// the reference's own call with its semantics (filter transform inside, synchronous); a second figure times
// the asynchronous surface (wino_conv_forward with pre-transformed filters), which is what tf32 / bf16 use.
// The reference reads pretrained weights and ImageNet batches (./vggData/conv*.bin, ./binImage/file_%d.bin);
// they are used if present, otherwise seeded synthetic tensors with the same shapes stand in.
// A host-side direct convolution of 2000 sampled outputs checks every result (the reference only checks that
// the first output is not exactly zero, comparison/layoutCompare.cu:219-226).
#include <cuda_bf16.h>

#include "cudnn_compare.h"
#include "harness_common.h"
#include "wino_compat.cuh"

using namespace harness;

int main(int argc, char** argv) {
    const int n = (int)arg_int(argc, argv, "batch", 8);
    const int opt = (int)arg_int(argc, argv, "opt", 1);
    const int layer = (int)arg_int(argc, argv, "layer", 6);
    const int iters = (int)arg_int(argc, argv, "iters", 20);
    const std::string dts0 = arg_str(argc, argv, "dtype", "fp32");
    const int wino = (int)arg_int(argc, argv, "wino", dts0 == "fp32" ? 4 : 0);
    const int check = (int)arg_int(argc, argv, "check", 1);
    const uint64_t seed = (uint64_t)arg_int(argc, argv, "seed", 0xC0DE);
    const std::string dts = arg_str(argc, argv, "dtype", "fp32");
    const int dtype = dts == "bf16" ? WINO_BF16 : dts == "tf32" ? WINO_TF32 : dts == "fp32x3" ? WINO_FP32X3 : WINO_FP32;
    const int cudnn_dtype = dtype == WINO_FP32X3 ? WINO_FP32 : dtype;   // FP32-accurate variants face cuDNN's CUDNN_FMA_MATH
    const int device = (int)arg_int(argc, argv, "device", 0);   // the reference hard-codes device 1 (layoutCompare.cu:33)
    LayerShape ls;
    if (!vgg_layer(layer, &ls) || opt < 0 || opt > 8) {
        printf("The layer is not right\n");
        return 1;
    }
    HCHECK_CUDA(cudaSetDevice(device));
    const int h = ls.h, c = ls.c, k = ls.k, pad = 1;
    printf("opt:%d\n", opt);

    // data: KCRS filters and NCHW images on the host, then permuted into the layout under test
    std::vector<float> w_kcrs((size_t)9 * k * c), x_nchw((size_t)n * c * h * h), bias(k, 0.f);
    if (!read_floats(ls.weights, w_kcrs.data(), w_kcrs.size())) fill_normal(w_kcrs.data(), w_kcrs.size(), seed + 1, std::sqrt(2.f / (9.f * c)));
    if (!read_floats("./binImage/file_0.bin", x_nchw.data(), x_nchw.size())) fill_uniform(x_nchw.data(), x_nchw.size(), seed, -1.f, 1.f);
    const int layout = opt <= 2 ? opt : (opt == 3 || opt == 4 || opt == 7) ? WINO_NCHW : WINO_NHWC;
    std::vector<float> x = to_layout(x_nchw, layout, n, c, h, h), w = filter_to_layout(w_kcrs, layout, k, c);
    if (dtype == WINO_BF16)   // the check compares against the values the kernels really see
        for (auto* v : {&x, &w})
            for (float& f : *v) f = __bfloat162float(__float2bfloat16(f));

    const size_t nx = x.size(), nw = w.size(), ny = (size_t)n * k * h * h;
    const size_t es = dtype == WINO_BF16 ? 2 : 4;
    void *xd, *wd, *yd;
    HCHECK_CUDA(cudaMalloc(&xd, nx * es));
    HCHECK_CUDA(cudaMalloc(&wd, nw * es));
    HCHECK_CUDA(cudaMalloc(&yd, ny * es));
    if (dtype == WINO_BF16) {
        std::vector<__nv_bfloat16> xb = to_bf16(x), wb = to_bf16(w);
        HCHECK_CUDA(cudaMemcpy(xd, xb.data(), nx * 2, cudaMemcpyHostToDevice));
        HCHECK_CUDA(cudaMemcpy(wd, wb.data(), nw * 2, cudaMemcpyHostToDevice));
    } else {
        HCHECK_CUDA(cudaMemcpy(xd, x.data(), nx * 4, cudaMemcpyHostToDevice));
        HCHECK_CUDA(cudaMemcpy(wd, w.data(), nw * 4, cudaMemcpyHostToDevice));
    }
    HCHECK_CUDA(cudaMemset(yd, 0, ny * es));

    cudaEvent_t e0, e1;
    HCHECK_CUDA(cudaEventCreate(&e0));
    HCHECK_CUDA(cudaEventCreate(&e1));
    std::vector<float> times;
    double fast_ms = -1;
    std::string note;

    if (opt <= 2) {
        wino_conv_desc d;
        memset(&d, 0, sizeof(d));
        d.layout_in = d.layout_out = layout;
        d.n = n; d.c = c; d.h = h; d.w = h; d.k = k; d.pad = pad; d.dtype = dtype; d.wino = wino;
        void *u, *ws;
        const size_t ub = wino_filter_bytes(&d), wsb = wino_conv_workspace_bytes(&d);
        if (!ub || !wsb) { fprintf(stderr, "libwino: %s\n", wino_last_error_string()); return 3; }
        HCHECK_CUDA(cudaMalloc(&u, ub));
        HCHECK_CUDA(cudaMalloc(&ws, wsb));
        if (dtype == WINO_FP32 && wino == 4) {
            // the reference's call: caller-owned workspaces of its minimum sizes (convModule_NCHW_padding.cu:44-50)
            const int bn = (h + 2 * pad - 2 + 3) / 4;
            const long long mp = ((long long)n * bn * bn + 127) / 128 * 128, np = (k + 127) / 128 * 128, kp = (c + 7) / 8 * 8;
            float *vt, *ut, *mt;
            HCHECK_CUDA(cudaMalloc(&vt, 36 * mp * kp * 4));
            HCHECK_CUDA(cudaMalloc(&ut, 36 * np * kp * 4));
            HCHECK_CUDA(cudaMalloc(&mt, 36 * mp * np * 4));
            warmup<<<1, 1>>>();
            float* out = (float*)yd;
            for (int i = 0; i < iters + 2; ++i) {
                int chn = c;
                HCHECK_CUDA(cudaEventRecord(e0));
                layoutManager((DataLayout)layout, (DataLayout)layout, n, h, chn, k, pad, (float*)xd, (float*)wd, vt, ut, mt, &out);
                HCHECK_CUDA(cudaDeviceSynchronize());
                HCHECK_CUDA(cudaEventRecord(e1));
                HCHECK_CUDA(cudaEventSynchronize(e1));
                float ms;
                HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
                if (i >= 2) times.push_back(ms);
            }
            cudaFree(vt); cudaFree(ut); cudaFree(mt);
            note = "layoutManager (reference call: filter transform inside, synchronous)";
        }
        // asynchronous surface: filters transformed once, forward timed back to back
        HCHECK_WINO(wino_filter_transform(&d, wd, u, nullptr));
        for (int i = 0; i < 3; ++i) HCHECK_WINO(wino_conv_forward(&d, xd, u, nullptr, yd, ws, wsb, nullptr));
        HCHECK_WINO(wino_device_status());
        if (times.empty()) {
            for (int i = 0; i < iters; ++i) {
                HCHECK_CUDA(cudaEventRecord(e0));
                HCHECK_WINO(wino_conv_forward(&d, xd, u, nullptr, yd, ws, wsb, nullptr));
                HCHECK_CUDA(cudaEventRecord(e1));
                HCHECK_CUDA(cudaEventSynchronize(e1));
                float ms;
                HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
                times.push_back(ms);
            }
            note = "wino_conv_forward (filters pre-transformed)";
        }
        HCHECK_CUDA(cudaEventRecord(e0));
        for (int i = 0; i < iters; ++i) HCHECK_WINO(wino_conv_forward(&d, xd, u, nullptr, yd, ws, wsb, nullptr));
        HCHECK_CUDA(cudaEventRecord(e1));
        HCHECK_CUDA(cudaEventSynchronize(e1));
        float ms;
        HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        fast_ms = ms / iters;
        HCHECK_WINO(wino_device_status());
        cudaFree(u); cudaFree(ws);
    } else {
        cudnnHandle_t handle;
        HCHECK_CUDNN(cudnnCreate(&handle));
        if (opt <= 6) {
            if (cudnn_dtype != WINO_FP32) { fprintf(stderr, "opt 3..6 are the reference's FP32 cuDNN modes; use opt 7/8 for %s\n", dts.c_str()); return 1; }
            cudnnTensorDescriptor_t xdesc, ydesc;
            cudnnFilterDescriptor_t wdesc;
            cudnnConvolutionDescriptor_t cdesc;
            HCHECK_CUDNN(cudnnCreateTensorDescriptor(&xdesc));
            HCHECK_CUDNN(cudnnCreateTensorDescriptor(&ydesc));
            HCHECK_CUDNN(cudnnCreateFilterDescriptor(&wdesc));
            HCHECK_CUDNN(cudnnCreateConvolutionDescriptor(&cdesc));
            printf("Conv_CuDNN\n");
            float* out = (float*)yd;
            for (int i = 0; i < iters + 2; ++i) {
                int chn = c;
                HCHECK_CUDA(cudaEventRecord(e0));
                const int rc = wino_cudnn_conv(n, h, chn, k, pad, (float*)xd, (float*)wd, &out, opt, handle, xdesc, ydesc, wdesc, cdesc);
                HCHECK_CUDA(cudaDeviceSynchronize());
                HCHECK_CUDA(cudaEventRecord(e1));
                HCHECK_CUDA(cudaEventSynchronize(e1));
                if (rc != 0) { printf("{\"opt\": %d, \"layer\": %d, \"unsupported\": true}\n", opt, layer); return 0; }
                float ms;
                HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
                if (i >= 2) times.push_back(ms);
            }
            note = "cuDNN legacy algorithm, FMA math";
        } else {
            const CudnnBest b = cudnn_best_forward(handle, opt == 7 ? CUDNN_TENSOR_NCHW : CUDNN_TENSOR_NHWC, cudnn_dtype, n, c, h, h, k, pad, xd, wd, yd, 5, iters);
            if (b.ms < 0) { printf("{\"opt\": %d, \"layer\": %d, \"unsupported\": true, \"tried\": \"%s\"}\n", opt, layer, b.tried.c_str()); return 0; }
            times.assign(iters, (float)b.ms);
            note = std::string("cuDNN best = ") + fwd_algo_name(b.algo) + " of [" + b.tried + "]";
        }
        cudnnDestroy(handle);
    }

    double sum = 0, best = 1e30;
    for (float t : times) {
        printf("time:%lf ms\n", (double)t);
        sum += t;
        best = t < best ? t : best;
    }
    const double avg = sum / times.size();
    const double flops = 2.0 * n * k * c * (double)h * h * 9;

    // D2H and check
    std::vector<float> y(ny);
    if (dtype == WINO_BF16) {
        std::vector<__nv_bfloat16> yb(ny);
        HCHECK_CUDA(cudaMemcpy(yb.data(), yd, ny * 2, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < ny; ++i) y[i] = __bfloat162float(yb[i]);
    } else {
        HCHECK_CUDA(cudaMemcpy(y.data(), yd, ny * 4, cudaMemcpyDeviceToHost));
    }
    printf("convOutput_cpu[0]:%lf\n", (double)y[0]);
    double err = -1;
    if (check) {
        err = spot_check(layout, layout, n, c, h, h, k, pad, x.data(), w.data(), nullptr, false, y.data(), 2000, seed + 7);
        const double tol = cudnn_dtype == WINO_FP32 ? 1e-4 : 2e-2;   // max-norm of sampled outputs; the L2 bars live in the test-suite
        if (!(err <= tol)) printf("moduleConv error\n");
    }
    printf("{\"harness\": \"layoutCompare\", \"opt\": %d, \"layer\": %d, \"batch\": %d, \"layout\": \"%s\", \"dtype\": \"%s\", \"c\": %d, "
           "\"k\": %d, \"h\": %d, \"ms_avg\": %.5f, \"ms_min\": %.5f, \"ms_async\": %.5f, \"tflops_direct_equiv\": %.2f, "
           "\"images_per_s\": %.1f, \"max_err_sampled\": %.3e, \"what\": \"%s\"}\n",
           opt, layer, n, layout_name(layout), dts.c_str(), c, k, h, avg, best, fast_ms, flops / (fast_ms > 0 ? fast_ms : avg) / 1e9,
           n / ((fast_ms > 0 ? fast_ms : avg) * 1e-3), err, note.c_str());
    cudaFree(xd); cudaFree(wd); cudaFree(yd);
    return 0;
}

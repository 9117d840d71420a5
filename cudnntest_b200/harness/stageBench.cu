// stageBench — per-stage micro-benchmark of the Winograd pipeline on the nine VGG-16 layer shapes.
//
// Takes the role of the reference's delayTest bench (delayTest/testbench/src/M1/M1TestBench_NCHW.cu:12-29: nine
// cases 224/1->64, 224/64->64, 112/64->128, 112/128->128, 56/128->256, 56/256->256, 28/256->512, 28/512->512,
// 14/512->512; M1Test.h:15-151: testValid against the host, testPerformance with min / max / avg delay;
// weightedSum :6-10), widened from its single kernel family (the input transform) to every stage of the path:
// input transform, tile GEMM (plain or row-fused), output transform, plus the whole convolution with the forced
// Winograd tile and with the engine's own choice of kernel.  Each stage is timed alone through the stage-level entry
// points of the C ABI, so a change to one kernel (tile shape, F(2x2) against F(4x4), operand format) shows up in
// its own column and in the weighted sum.
//
//   stageBench batch=B layout=nchw|nhwc|chwn dtype=fp32|fp32x3|tf32|bf16 wino=4|2 iters=20 hbm=<GB/s> tflops=<TFLOP/s>
//
// Per case it prints one line per stage: avg / min / max microseconds, algorithmic GB/s (or TFLOP/s for the GEMM) and
// the fraction of the peak given on the command line (defaults: the HBM copy bandwidth and the sustained BF16 GEMM
// rate measured on this pool's B200, 6538.6 GB/s and 1351.9 TFLOP/s; pass tflops= for TF32 / FP32).  "valid" is a
// host-side spot check of 500 sampled outputs of the staged pipeline.  The last lines are the weighted sums: with
// the reference's weights (1,1,1,1,1,3,1,3,4) and with VGG-16's layer multiplicities (1,1,1,1,1,2,1,2,3).
#include <algorithm>

#include "harness_common.h"

using namespace harness;

struct Case { int side, c, k; };
static const Case kCases[9] = {{224, 3, 64},  {224, 64, 64},  {112, 64, 128}, {112, 128, 128}, {56, 128, 256},
                               {56, 256, 256}, {28, 256, 512}, {28, 512, 512}, {14, 512, 512}};

struct Timing { double avg = 0, mn = 0, mx = 0; };

template <typename F>
static Timing time_stage(int iters, F&& launch) {
    cudaEvent_t e0, e1;
    HCHECK_CUDA(cudaEventCreate(&e0));
    HCHECK_CUDA(cudaEventCreate(&e1));
    for (int i = 0; i < 3; ++i) launch();
    HCHECK_CUDA(cudaDeviceSynchronize());
    Timing t;
    t.mn = 1e30;
    for (int i = 0; i < iters; ++i) {
        HCHECK_CUDA(cudaEventRecord(e0));
        launch();
        HCHECK_CUDA(cudaEventRecord(e1));
        HCHECK_CUDA(cudaEventSynchronize(e1));
        float ms;
        HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        const double us = ms * 1e3;
        t.avg += us / iters;
        t.mn = std::min(t.mn, us);
        t.mx = std::max(t.mx, us);
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return t;
}

int main(int argc, char** argv) {
    const int n = (int)arg_int(argc, argv, "batch", 1);      // the reference's cases use batch 1
    const int iters = (int)arg_int(argc, argv, "iters", 20);
    const int wino = (int)arg_int(argc, argv, "wino", 4);
    const std::string dts = arg_str(argc, argv, "dtype", "bf16"), los = arg_str(argc, argv, "layout", "nhwc");
    const int dtype = dts == "bf16" ? WINO_BF16 : dts == "tf32" ? WINO_TF32 : dts == "fp32x3" ? WINO_FP32X3 : WINO_FP32;
    const int layout = los == "nchw" ? WINO_NCHW : los == "chwn" ? WINO_CHWN : WINO_NHWC;
    const double hbm = atof(arg_str(argc, argv, "hbm", "6538.6").c_str());
    const double tpeak = atof(arg_str(argc, argv, "tflops", "1351.9").c_str());
    if ((wino != 2 && wino != 4) || n <= 0) { fprintf(stderr, "wino must be 2 or 4, batch positive\n"); return 1; }
    HCHECK_CUDA(cudaSetDevice((int)arg_int(argc, argv, "device", 0)));
    const size_t es = dtype == WINO_BF16 ? 2 : 4;
    const int a = wino + 2;
    double total_us[9], engine_us[9];
    bool all_valid = true;

    for (int ci = 0; ci < 9; ++ci) {
        const Case& cs = kCases[ci];
        const int h = cs.side, c = cs.c, k = cs.k, pad = 1;
        std::vector<float> x_nchw((size_t)n * c * h * h), w_kcrs((size_t)9 * k * c), bias(k);
        fill_uniform(x_nchw.data(), x_nchw.size(), 11 + ci, -1.f, 1.f);
        fill_normal(w_kcrs.data(), w_kcrs.size(), 31 + ci, std::sqrt(2.f / (9.f * c)));
        fill_normal(bias.data(), bias.size(), 51 + ci, 0.01f);
        std::vector<float> x = to_layout(x_nchw, layout, n, c, h, h), w = filter_to_layout(w_kcrs, layout, k, c);
        if (dtype == WINO_BF16)
            for (auto* v : {&x, &w})
                for (float& f : *v) f = __bfloat162float(__float2bfloat16(f));
        const size_t ny = (size_t)n * k * h * h;
        void *xd, *wd, *yd;
        float* bd;
        HCHECK_CUDA(cudaMalloc(&xd, x.size() * es));
        HCHECK_CUDA(cudaMalloc(&wd, w.size() * es));
        HCHECK_CUDA(cudaMalloc(&yd, ny * es));
        HCHECK_CUDA(cudaMalloc(&bd, k * sizeof(float)));
        HCHECK_CUDA(cudaMemcpy(bd, bias.data(), k * sizeof(float), cudaMemcpyHostToDevice));
        if (dtype == WINO_BF16) {
            auto xb = to_bf16(x), wb = to_bf16(w);
            HCHECK_CUDA(cudaMemcpy(xd, xb.data(), xb.size() * 2, cudaMemcpyHostToDevice));
            HCHECK_CUDA(cudaMemcpy(wd, wb.data(), wb.size() * 2, cudaMemcpyHostToDevice));
        } else {
            HCHECK_CUDA(cudaMemcpy(xd, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
            HCHECK_CUDA(cudaMemcpy(wd, w.data(), w.size() * 4, cudaMemcpyHostToDevice));
        }

        wino_conv_desc d;
        memset(&d, 0, sizeof(d));
        d.layout_in = layout; d.layout_out = layout; d.n = n; d.c = c; d.h = h; d.w = h; d.k = k; d.pad = pad;
        d.dtype = dtype; d.wino = wino; d.relu = 1; d.has_bias = 1;
        d.slab_images = n;                                    // stages run on the whole batch as one slab
        const long long tp = wino_stage_tile_rows(&d, n);
        const int cp = wino_stage_cp(&d), kq = wino_stage_kq(&d);
        if (tp <= 0 || cp <= 0 || kq <= 0) { fprintf(stderr, "libwino: %s\n", wino_last_error_string()); return 3; }
        const bool fused = dtype == WINO_TF32 || dtype == WINO_BF16;              // tensor-core variants have the row-fused pair of stages
        const size_t op_es = dtype == WINO_BF16 ? 2 : 4;
        const size_t v_bytes = (size_t)a * a * tp * cp * op_es;
        const size_t m_bytes = (size_t)a * a * tp * kq * 4;  // large enough for the raw products and for Z
        void *u, *v, *m;
        HCHECK_CUDA(cudaMalloc(&u, wino_filter_bytes(&d)));
        HCHECK_CUDA(cudaMalloc(&v, v_bytes));
        HCHECK_CUDA(cudaMalloc(&m, m_bytes));
        HCHECK_WINO(wino_filter_transform(&d, wd, u, nullptr));

        const Timing t_in = time_stage(iters, [&] { HCHECK_WINO(wino_stage_input_transform(&d, xd, 0, n, v, nullptr)); });
        const Timing t_g = time_stage(iters, [&] { HCHECK_WINO(wino_stage_gemm(&d, v, u, (float*)m, n, nullptr)); });
        const Timing t_out = time_stage(iters, [&] { HCHECK_WINO(wino_stage_output_transform(&d, (const float*)m, bd, yd, 0, n, nullptr)); });
        // validity of the staged pipeline: sampled outputs against a host-side direct convolution
        std::vector<float> y(ny);
        if (dtype == WINO_BF16) {
            std::vector<__nv_bfloat16> yb(ny);
            HCHECK_CUDA(cudaMemcpy(yb.data(), yd, ny * 2, cudaMemcpyDeviceToHost));
            for (size_t i = 0; i < ny; ++i) y[i] = __bfloat162float(yb[i]);
        } else {
            HCHECK_CUDA(cudaMemcpy(y.data(), yd, ny * 4, cudaMemcpyDeviceToHost));
        }
        const double err = spot_check(layout, layout, n, c, h, h, k, pad, x.data(), w.data(), bias.data(), true, y.data(), 500, 77 + ci);
        const bool valid = err <= (dtype == WINO_FP32 || dtype == WINO_FP32X3 ? 1e-4 : 2e-2);
        all_valid = all_valid && valid;
        Timing t_gz, t_oz;
        if (fused) {
            t_gz = time_stage(iters, [&] { HCHECK_WINO(wino_stage_gemm_rowfused(&d, v, u, m, n, nullptr)); });
            t_oz = time_stage(iters, [&] { HCHECK_WINO(wino_stage_output_transform_rowfused(&d, m, bd, yd, 0, n, nullptr)); });
        }
        HCHECK_WINO(wino_device_status());

        // whole convolution: forced Winograd tile, then the engine's own choice of kernel
        void* ws;
        const size_t wsb = wino_conv_workspace_bytes(&d);
        HCHECK_CUDA(cudaMalloc(&ws, wsb));
        d.slab_images = 0;
        const Timing t_conv = time_stage(iters, [&] { HCHECK_WINO(wino_conv_forward(&d, xd, u, bd, yd, ws, wsb, nullptr)); });
        cudaFree(ws); cudaFree(u);
        wino_conv_desc de = d;
        de.wino = 0;
        void *ue, *wse;
        const size_t wsbe = wino_conv_workspace_bytes(&de);
        HCHECK_CUDA(cudaMalloc(&ue, wino_filter_bytes(&de)));
        HCHECK_CUDA(cudaMalloc(&wse, wsbe));
        HCHECK_WINO(wino_filter_transform(&de, wd, ue, nullptr));
        const Timing t_eng = time_stage(iters, [&] { HCHECK_WINO(wino_conv_forward(&de, xd, ue, bd, yd, wse, wsbe, nullptr)); });
        HCHECK_WINO(wino_device_status());

        // algorithmic bytes / flops of each stage (unpadded tile count T)
        const long long bn = (h + wino - 1) / wino;
        const double T = (double)n * bn * bn;
        const double b_in = (double)n * c * h * h * es + (double)a * a * T * c * op_es;
        const double f_g = 2.0 * a * a * T * c * k;
        const double b_out = (double)a * a * T * k * 4 + (double)n * k * h * h * es;
        const double b_oz = (double)a * wino * T * k * (dtype == WINO_BF16 ? 2 : 4) + (double)n * k * h * h * es;
        const double f_conv = 2.0 * n * k * c * (double)h * h * 9;
        printf("case %d: side %d  %d -> %d  batch %d  %s %s F(%dx%d,3x3)  valid=%s (max err %.2e)\n", ci + 1, h, c, k, n, layout_name(layout),
               dts.c_str(), wino, wino, valid ? "yes" : "NO", err);
        auto line = [&](const char* name, const Timing& t, double bytes, double flops) {
            printf("  %-28s avg %9.2f us  min %9.2f  max %9.2f", name, t.avg, t.mn, t.mx);
            if (bytes > 0) printf("  %8.1f GB/s (%.2f of %.0f)", bytes / t.avg / 1e3, bytes / t.avg / 1e3 / hbm, hbm);
            if (flops > 0) printf("  %8.1f TFLOP/s (%.2f of %.0f)", flops / t.avg / 1e6, flops / t.avg / 1e6 / tpeak, tpeak);
            printf("\n");
        };
        line("input transform", t_in, b_in, 0);
        line("tile GEMM (products M)", t_g, 0, f_g);
        line("output transform (from M)", t_out, b_out, 0);
        if (fused) {
            line("tile GEMM (row-fused, Z)", t_gz, 0, f_g);
            line("output transform (from Z)", t_oz, b_oz, 0);
        }
        line("convolution, forced Winograd", t_conv, 0, f_conv);
        line("convolution, engine's choice", t_eng, 0, f_conv);
        total_us[ci] = t_conv.avg;
        engine_us[ci] = t_eng.avg;
        cudaFree(ue); cudaFree(wse); cudaFree(v); cudaFree(m);
        cudaFree(xd); cudaFree(wd); cudaFree(yd); cudaFree(bd);
    }
    // weightedSum (M1TestBench_NCHW.cu:6-10) and the same with VGG-16's own layer multiplicities
    static const int w_ref[9] = {1, 1, 1, 1, 1, 3, 1, 3, 4}, w_vgg[9] = {1, 1, 1, 1, 1, 2, 1, 2, 3};
    double s_ref = 0, s_vgg = 0, e_ref = 0, e_vgg = 0;
    for (int i = 0; i < 9; ++i) {
        s_ref += w_ref[i] * total_us[i]; s_vgg += w_vgg[i] * total_us[i];
        e_ref += w_ref[i] * engine_us[i]; e_vgg += w_vgg[i] * engine_us[i];
    }
    printf("totalTime:%f\n", s_ref);
    printf("{\"harness\": \"stageBench\", \"batch\": %d, \"layout\": \"%s\", \"dtype\": \"%s\", \"wino\": %d, \"valid\": %s, "
           "\"weighted_us_reference_weights\": %.2f, \"weighted_us_vgg16\": %.2f, \"engine_weighted_us_reference_weights\": %.2f, "
           "\"engine_weighted_us_vgg16\": %.2f}\n",
           n, layout_name(layout), dts.c_str(), wino, all_valid ? "true" : "false", s_ref, s_vgg, e_ref, e_vgg);
    return all_valid ? 0 : 2;
}

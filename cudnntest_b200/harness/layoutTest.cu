// layoutTest — single-convolution driver: N H C K on the command line, ten timed calls, result dumped as raw
// float32 for offline comparison.
//
// Takes the role of layoutTest/{NCHW,NHWC,CHWN}/convModule_<L>_padding.cu (main at convModule_NCHW_padding.cu:7-115):
// positional arguments N H C K (:19-22), padding 1, input and filters from data/input.bin and data/filter.bin if
// present (the notebooks write them, ConvTest_V3_NCHW-Mar18.ipynb cell 1) else seeded rand()-0.5 values like the
// notebooks use, exact-size workspaces (:48-72), 10 timed wrapedConv_<L> calls between two events (:79-89), the
// reference's own print "time ... us  ... TFLOPS" with its MAC-count formula ((9C)C + C)H^2 N (:95), the first
// output, and data/ConvModule_<L>.bin (:108-112).  layout=NCHW|NHWC|CHWN selects which of the three programs
// this run stands for.  A true FLOP rate and a sampled check against a host direct convolution are added.
#include "harness_common.h"
#include "wino_compat.cuh"

using namespace harness;

int main(int argc, char** argv) {
    if (argc < 5) {
        fprintf(stderr, "usage: %s N H C K [layout=NCHW|NHWC|CHWN] [dir=data] [device=0]\n", argv[0]);
        return 1;
    }
    const int n = atoi(argv[1]), h = atoi(argv[2]), c = atoi(argv[3]), k = atoi(argv[4]), pad = 1;
    const std::string ls = arg_str(argc, argv, "layout", "NCHW"), dir = arg_str(argc, argv, "dir", "data");
    const int layout = ls == "NHWC" ? WINO_NHWC : ls == "CHWN" ? WINO_CHWN : WINO_NCHW;
    HCHECK_CUDA(cudaSetDevice((int)arg_int(argc, argv, "device", 0)));
    if (n <= 0 || h <= 0 || c <= 0 || k <= 0) { fprintf(stderr, "bad shape\n"); return 1; }

    std::vector<float> x((size_t)n * c * h * h), w((size_t)9 * k * c);
    if (!read_floats((dir + "/input.bin").c_str(), x.data(), x.size())) fill_uniform(x.data(), x.size(), 11, -0.5f, 0.5f);
    if (!read_floats((dir + "/filter.bin").c_str(), w.data(), w.size())) fill_uniform(w.data(), w.size(), 12, -0.5f, 0.5f);
    // the files hold the tensors already in the layout under test (the notebooks write them that way)

    const int oside = h + 2 * pad - 2, bn = (oside + 3) / 4;
    const long long mp = ((long long)n * bn * bn + 127) / 128 * 128, np = (k + 127) / 128 * 128, kp = (c + 7) / 8 * 8;
    float *xd, *wd, *yd, *vt, *ut, *mt;
    const size_t ny = (size_t)n * k * oside * oside;
    HCHECK_CUDA(cudaMalloc(&xd, x.size() * 4));
    HCHECK_CUDA(cudaMalloc(&wd, w.size() * 4));
    HCHECK_CUDA(cudaMalloc(&yd, ny * 4));
    HCHECK_CUDA(cudaMalloc(&vt, 36 * mp * kp * 4));
    HCHECK_CUDA(cudaMalloc(&ut, 36 * np * kp * 4));
    HCHECK_CUDA(cudaMalloc(&mt, 36 * mp * np * 4));
    HCHECK_CUDA(cudaMemcpy(xd, x.data(), x.size() * 4, cudaMemcpyHostToDevice));
    HCHECK_CUDA(cudaMemcpy(wd, w.data(), w.size() * 4, cudaMemcpyHostToDevice));

    warmup<<<1, 1>>>();
    int chn = c;
    layoutManager((DataLayout)layout, (DataLayout)layout, n, h, chn, k, pad, xd, wd, vt, ut, mt, &yd);   // untimed first call
    cudaEvent_t e0, e1;
    HCHECK_CUDA(cudaEventCreate(&e0));
    HCHECK_CUDA(cudaEventCreate(&e1));
    HCHECK_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < 10; ++i) {
        chn = c;
        layoutManager((DataLayout)layout, (DataLayout)layout, n, h, chn, k, pad, xd, wd, vt, ut, mt, &yd);
    }
    HCHECK_CUDA(cudaEventRecord(e1));
    HCHECK_CUDA(cudaEventSynchronize(e1));
    float ms;
    HCHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    const double us = ms * 1e3 / 10;
    const double ref_macs = ((9.0 * c) * c + c) * (double)h * h * n;              // the reference's formula (K taken as C)
    const double flops = 2.0 * n * k * c * (double)oside * oside * 9;
    printf("time %f us  %f TFLOPS\n", us, ref_macs / us * 1e-6);
    printf("true rate %f TFLOP/s (2*N*K*C*OH*OW*9)\n", flops / us * 1e-6);

    std::vector<float> y(ny);
    HCHECK_CUDA(cudaMemcpy(y.data(), yd, ny * 4, cudaMemcpyDeviceToHost));
    printf("output_cpu[0]:%f\n", y[0]);
    if (y[0] == 0.0f) printf("moduleConv error\n");
    const double err = spot_check(layout, layout, n, c, h, h, k, pad, x.data(), w.data(), nullptr, false, y.data(), 2000, 99);
    printf("sampled max|err|/max|ref| vs host direct convolution: %.3e %s\n", err, err <= 1e-4 ? "(ok)" : "(moduleConv error)");
    const std::string out = dir + "/ConvModule_" + ls + ".bin";
    if (!write_floats(out.c_str(), y.data(), ny)) printf("(result not saved: cannot write %s)\n", out.c_str());
    return err <= 1e-4 ? 0 : 5;
}

// Helpers of the harness executables: key=value command line, raw float32 file IO, seeded synthetic tensors,
// a host-side direct convolution for spot checks, error macros.  Original code; the reference uses NVIDIA's
// sample header error_util.h (comparison/error_util.h) and util.h:99-127 for the same jobs.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "wino.h"

#define HCHECK_CUDA(expr)                                                                              \
    do {                                                                                               \
        cudaError_t e_ = (expr);                                                                       \
        if (e_ != cudaSuccess) {                                                                       \
            fprintf(stderr, "%s:%d: %s failed: %s\n", __FILE__, __LINE__, #expr, cudaGetErrorString(e_)); \
            exit(2);                                                                                   \
        }                                                                                              \
    } while (0)

#define HCHECK_WINO(expr)                                                                          \
    do {                                                                                           \
        int rc_ = (expr);                                                                          \
        if (rc_ != WINO_OK) {                                                                      \
            fprintf(stderr, "%s:%d: %s failed (%d): %s\n", __FILE__, __LINE__, #expr, rc_, wino_last_error_string()); \
            exit(3);                                                                               \
        }                                                                                          \
    } while (0)

namespace harness {

// "name=value" anywhere on the command line (the reference's spelling: batch=8 opt=1 layer=6); default if absent
inline long arg_int(int argc, char** argv, const char* name, long dflt) {
    const size_t n = strlen(name);
    for (int i = 1; i < argc; ++i) {
        const char* a = argv[i];
        while (*a == '-') ++a;
        if (strncmp(a, name, n) == 0 && a[n] == '=') return atol(a + n + 1);
    }
    return dflt;
}
inline std::string arg_str(int argc, char** argv, const char* name, const char* dflt) {
    const size_t n = strlen(name);
    for (int i = 1; i < argc; ++i) {
        const char* a = argv[i];
        while (*a == '-') ++a;
        if (strncmp(a, name, n) == 0 && a[n] == '=') return std::string(a + n + 1);
    }
    return dflt;
}

// raw little-endian float32 files, the reference's .bin format
inline bool read_floats(const char* path, float* dst, size_t count) {
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    const size_t got = fread(dst, sizeof(float), count, f);
    fclose(f);
    return got == count;
}
inline bool write_floats(const char* path, const float* src, size_t count) {
    FILE* f = fopen(path, "wb");
    if (!f) return false;
    const size_t put = fwrite(src, sizeof(float), count, f);
    fclose(f);
    return put == count;
}

// counter-based generator: splitmix64 of (seed, index)
inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
inline double unit(uint64_t seed, uint64_t i) { return (double)(mix64(seed * 0x100000001B3ull + i) >> 11) * (1.0 / 9007199254740992.0); }
inline void fill_uniform(float* p, size_t n, uint64_t seed, float lo, float hi) {
    for (size_t i = 0; i < n; ++i) p[i] = lo + (hi - lo) * (float)unit(seed, i);
}
inline void fill_normal(float* p, size_t n, uint64_t seed, float sigma) {
    for (size_t i = 0; i < n; ++i) {
        const double u1 = unit(seed, 2 * i) + 1e-300, u2 = unit(seed, 2 * i + 1);
        p[i] = sigma * (float)(std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586 * u2));
    }
}

struct Strides4 { long long n, c, h, w; };
inline Strides4 act_strides(int layout, long long N, long long C, long long H, long long W) {
    if (layout == WINO_NCHW) return {C * H * W, H * W, W, 1};
    if (layout == WINO_NHWC) return {H * W * C, 1, W * C, C};
    return {1, H * W * N, W * N, N};
}
inline Strides4 flt_strides(int layout, long long K, long long C) {
    if (layout == WINO_NCHW) return {C * 9, 9, 3, 1};
    if (layout == WINO_NHWC) return {9 * C, 1, 3 * C, C};
    return {1, 9 * K, 3 * K, K};
}

// Host-side direct convolution of `samples` pseudo-randomly chosen outputs, double accumulation; returns the
// largest |y - ref| / max|ref| over the samples (x, w, y in the given layouts; y before any pooling).
inline double spot_check(int layout_in, int layout_out, int N, int C, int H, int W, int K, int pad, const float* x,
                         const float* w, const float* bias, bool relu, const float* y, int samples, uint64_t seed) {
    const int OH = H + 2 * pad - 2, OW = W + 2 * pad - 2;
    const Strides4 sx = act_strides(layout_in, N, C, H, W), sw = flt_strides(layout_in, K, C), sy = act_strides(layout_out, N, K, OH, OW);
    double worst = 0, scale = 1e-30;
    for (int i = 0; i < samples; ++i) {
        const int n = (int)(mix64(seed + 4 * i) % N), k = (int)(mix64(seed + 4 * i + 1) % K);
        const int oh = (int)(mix64(seed + 4 * i + 2) % OH), ow = (int)(mix64(seed + 4 * i + 3) % OW);
        double acc = bias ? bias[k] : 0.0;
        for (int c = 0; c < C; ++c)
            for (int r = 0; r < 3; ++r)
                for (int s = 0; s < 3; ++s) {
                    const int ih = oh + r - pad, iw = ow + s - pad;
                    if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                    acc += (double)x[n * sx.n + c * sx.c + ih * sx.h + iw * sx.w] * (double)w[k * sw.n + c * sw.c + r * sw.h + s * sw.w];
                }
        if (relu && acc < 0) acc = 0;
        const double got = y[n * sy.n + k * sy.c + oh * sy.h + ow * sy.w];
        worst = std::fmax(worst, std::fabs(got - acc));
        scale = std::fmax(scale, std::fabs(acc));
    }
    return worst / scale;
}

inline std::vector<float> to_layout(const std::vector<float>& nchw, int layout, int N, int C, int H, int W) {
    std::vector<float> out(nchw.size());
    const Strides4 s = act_strides(layout, N, C, H, W);
    size_t i = 0;
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c)
            for (int h = 0; h < H; ++h)
                for (int w = 0; w < W; ++w) out[n * s.n + c * s.c + h * s.h + w * s.w] = nchw[i++];
    return out;
}
inline std::vector<float> filter_to_layout(const std::vector<float>& kcrs, int layout, int K, int C) {
    std::vector<float> out(kcrs.size());
    const Strides4 s = flt_strides(layout, K, C);
    size_t i = 0;
    for (int k = 0; k < K; ++k)
        for (int c = 0; c < C; ++c)
            for (int r = 0; r < 3; ++r)
                for (int q = 0; q < 3; ++q) out[k * s.n + c * s.c + r * s.h + q * s.w] = kcrs[i++];
    return out;
}

inline std::vector<__nv_bfloat16> to_bf16(const std::vector<float>& v) {
    std::vector<__nv_bfloat16> o(v.size());
    for (size_t i = 0; i < v.size(); ++i) o[i] = __float2bfloat16(v[i]);
    return o;
}

// the nine VGG-16 layer shapes of the reference's per-layer benchmark (comparison/layoutCompare.cu:41-82)
struct LayerShape { int h, c, k; const char* weights; };
inline bool vgg_layer(int layer, LayerShape* s) {
    static const LayerShape t[9] = {{224, 3, 64, "./vggData/conv1.bin"},   {224, 64, 64, "./vggData/conv2.bin"},
                                    {112, 64, 128, "./vggData/conv3.bin"}, {112, 128, 128, "./vggData/conv4.bin"},
                                    {56, 128, 256, "./vggData/conv5.bin"}, {56, 256, 256, "./vggData/conv7.bin"},
                                    {28, 256, 512, "./vggData/conv8.bin"}, {28, 512, 512, "./vggData/conv10.bin"},
                                    {14, 512, 512, "./vggData/conv13.bin"}};
    if (layer < 1 || layer > 9) return false;
    *s = t[layer - 1];
    return true;
}

inline const char* layout_name(int l) { return l == WINO_NCHW ? "NCHW" : l == WINO_NHWC ? "NHWC" : "CHWN"; }

}  // namespace harness

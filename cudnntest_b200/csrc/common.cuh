// Shared definitions of libwino's translation units: element types, layout strides, the problem
// geometry derived from a wino_conv_desc, error reporting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "../../include/wino.h"

namespace wino {

// ---- element types -----------------------------------------------------------------------------------
// A float that has been rounded to the TF32 grid (10 explicit mantissa bits) when stored.
struct tf32_t {
    float v;
};

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<tf32_t>(tf32_t v) { return v.v; }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ tf32_t from_float<tf32_t>(float v) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(v));
    tf32_t t;
    t.v = __uint_as_float(r);
    return t;
}

// Split operand of the FP32X3 variant: a float x is used as two TF32 values, head hi = tf32(x) and tail
// lo = tf32(x - hi).  The transformed filters are stored that way (head at column c, tail at column Cp + c of a row
// of 2*Cp floats); the transformed input tiles are split inside the tile GEMM.
struct tf32x2_t {
    float hi, lo;
};
__device__ __forceinline__ tf32x2_t split_tf32(float v) {
    tf32x2_t r;
    r.hi = from_float<tf32_t>(v).v;
    r.lo = from_float<tf32_t>(v - r.hi).v;
    return r;
}

// ---- layouts -----------------------------------------------------------------------------------------
struct Strides {
    long long n, c, h, w;
};

// element strides of an activation tensor with logical dims (N, C, H, W) stored in `layout`
__host__ __device__ inline Strides act_strides(int layout, long long N, long long C, long long H, long long W) {
    Strides s;
    if (layout == WINO_NCHW) { s.n = C * H * W; s.c = H * W; s.h = W; s.w = 1; }
    else if (layout == WINO_NHWC) { s.n = H * W * C; s.c = 1; s.h = W * C; s.w = C; }
    else { s.n = 1; s.c = H * W * N; s.h = W * N; s.w = N; }
    return s;
}

// element strides of the 3x3 filter tensor as (k, c, r, s); the filter layout follows the input layout
__host__ __device__ inline Strides filter_strides(int layout, long long K, long long C) {
    Strides s;
    if (layout == WINO_NCHW) { s.n = C * 9; s.c = 9; s.h = 3; s.w = 1; }        // KCRS
    else if (layout == WINO_NHWC) { s.n = 9 * C; s.c = 1; s.h = 3 * C; s.w = C; } // KRSC
    else { s.n = 1; s.c = 9 * K; s.h = 3 * K; s.w = K; }                          // CRSK
    return s;
}

// ---- geometry ----------------------------------------------------------------------------------------
enum OperandKind { OP_F32 = 0, OP_TF32 = 1, OP_BF16 = 2, OP_F16 = 3, OP_TF32X3 = 4 };

struct Geometry {
    int m;            // output tile side (2 or 4)
    int a;            // input tile side m + 2
    int oh, ow;       // conv output size before pooling
    int ph, pw;       // stored output size (after optional pool)
    int bny, bnx;     // tiles per image
    int tiles_img;    // bny * bnx
    int cp;           // channels padded to 8 (zero filled): the contraction length of the tile GEMM
    int crow;         // U row length in elements: cp, or 2*cp for OP_TF32X3 (cp TF32 heads, then cp TF32 tails); V rows are always cp
    int kq;           // M row length
    int operand;      // OperandKind of V and U
    int esize_io;     // bytes per activation element of x
    int out_bf16;     // y is stored as bfloat16 (else float)
    int esize_op;     // bytes per V/U element
    int prod_kind;    // what the tile GEMM of wino_conv_forward writes: 0 = M (float), 1 = Z (float), 2 = Z (half)
    int prod_planes;  // a*a for M, a*m for Z
    int esize_prod;   // bytes per product element
};

inline int round_up(int x, int q) { return (x + q - 1) / q * q; }
inline long long round_up_ll(long long x, long long q) { return (x + q - 1) / q * q; }

// y stored in another element type than x: such layers always run the Winograd pipeline, whose output transform converts
inline bool out_type_differs(const wino_conv_desc& d) {
    return (d.out_dtype == WINO_OUT_FP32 && d.dtype == WINO_BF16) || (d.out_dtype == WINO_OUT_BF16 && d.dtype != WINO_BF16);
}

// ---- errors ------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define WINO_CUDA_CHECK(expr)                                                                     \
    do {                                                                                          \
        cudaError_t _e = (expr);                                                                  \
        if (_e != cudaSuccess)                                                                    \
            return ::wino::fail(WINO_E_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                                __FILE__, __LINE__);                                              \
    } while (0)

// ---- host helpers shared by the entry points (defined in api.cu) --------------------------------------
int make_geometry(const wino_conv_desc* d, Geometry* g);   // validates the descriptor, derives the tiling
long long per_image_bytes(const Geometry& g);              // V + M bytes one image contributes to a slab
long long tile_rows(const Geometry& g, int ns);            // rows per V/M plane for a slab of ns images
size_t v_bytes(const Geometry& g, long long tp);
size_t m_bytes(const Geometry& g, long long tp);          // raw product buffer M (stage-level entry points)
size_t prod_bytes(const Geometry& g, long long tp);       // product buffer of wino_conv_forward (M or Z)
int run_conv_gemm(const Geometry& g, const void* v, const void* u, void* prod, int k, long long t_rows, long long tp,
                  cudaStream_t st);
int run_gemm(const Geometry& g, const void* v, const void* u, float* m, int k, long long t_rows, long long tp,
             cudaStream_t st);
int check_device();
size_t wino_u_bytes(const wino_conv_desc& d, const Geometry& g);          // transformed filters U
size_t direct_filter_offset(const wino_conv_desc& d, const Geometry& g);  // start of the packed filters when the buffer holds both
const void* direct_filters(const wino_conv_desc& d, const Geometry& g, const void* u);   // what the direct kernels read

// ---- measurement hooks -----------------------------------------------------------------------------------
void count_launch();
enum Stage { STAGE_INPUT = 0, STAGE_GEMM = 1, STAGE_OUTPUT = 2, STAGE_FILTER = 3, STAGE_GEMM_ROWFUSED = 4, STAGE_DIRECT = 5, STAGE_DIRECT_TC = 6, STAGE_COUNT = 8 };
// brackets one kernel launch with CUDA events when profiling is enabled
struct ProfScope {
    ProfScope(int stage, cudaStream_t st);
    ~ProfScope();
    int slot;
    cudaStream_t st;
};

// ---- kernel launchers (one per translation unit) -------------------------------------------------------
int launch_filter_transform(const wino_conv_desc& d, const Geometry& g, const void* w, void* u, cudaStream_t st);
int launch_input_transform(const wino_conv_desc& d, const Geometry& g, const void* x, int n0, int ns, void* v,
                           long long tp, cudaStream_t st);
// prod_kind: 0 = raw products M[a*a] (float), 1 = row-transformed Z[a*m] (float), 2 = Z (half), 3 = raw products in
// 3 bytes (plane of upper 16 bits at m, plane of third bytes behind it; NHWC destinations: output_transform_m24_ok)
int launch_output_transform(const wino_conv_desc& d, const Geometry& g, const void* m, int prod_kind, const float* bias,
                            void* y, int n0, int ns, long long tp, cudaStream_t st);
bool output_transform_m24_ok(const wino_conv_desc& d, const void* y);
int launch_gemm_ffma(const float* v, const float* u, float* m, int batches, long long t_rows, long long tp, int k,
                     int cp, int kq, cudaStream_t st);
// direct convolution on tensor cores for thin, large-spatial NHWC BF16 layers, C = 64 / 128 (direct_tc.cu)
bool direct_tc_applies(const wino_conv_desc& d);
// What the filter buffer of this descriptor holds, whatever its batch size: 0 = transformed filters U only, 1 = filters
// packed for the direct kernel only, 2 = U followed (on a 1 KiB boundary) by the packed filters, because the engine
// picks between the two kernels by batch size (NHWC directly, the other layouts through NHWC staging).
int direct_filter_mode(const wino_conv_desc& d);
size_t direct_tc_filter_bytes(const wino_conv_desc& d);
int launch_direct_tc_pack(const wino_conv_desc& d, const void* w, void* packed, cudaStream_t st);
// y_nchw: store the result NCHW although d says NHWC (only where direct_tc_stores_nchw(d), direct_tc.cuh)
int launch_direct_tc(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                     cudaStream_t st, bool y_nchw = false);
// BF16 / TF32 layers in NCHW / CHWN whose NHWC twin takes the direct kernel: the activations are relaid out to NHWC
// staging buffers around the direct kernel (extra passes over x and y cost less HBM time than the Winograd pipeline's
// transform-domain buffers); an NCHW result is stored by the filters-as-M kernel itself, without a pass over y.
// staging bytes = what `scratch` must hold; the filters are packed as for the direct kernel.
bool direct_via_nhwc_applies(const wino_conv_desc& d);
size_t direct_via_nhwc_staging_bytes(const wino_conv_desc& d, const Geometry& g);
int launch_direct_via_nhwc(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias, void* y,
                           void* scratch, size_t scratch_bytes, cudaStream_t st);
// thin-input (C <= 3) direct convolution on tensor cores (direct_small_c.cu)
bool direct_small_c_applies(const wino_conv_desc& d);
size_t direct_small_c_filter_bytes(const wino_conv_desc& d);
int launch_direct_small_c_pack(const wino_conv_desc& d, const void* w, void* packed, cudaStream_t st);
int launch_direct_small_c(const wino_conv_desc& d, const Geometry& g, const void* x, const void* packed, const float* bias,
                          void* y, cudaStream_t st);
int launch_relayout(int src, int dst, int n, int c, int h, int w, int esize, const void* in, void* out,
                    cudaStream_t st);
int launch_maxpool(int layout, int n, int c, int h, int w, int dtype, const void* in, void* out, cudaStream_t st);

}  // namespace wino

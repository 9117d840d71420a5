/* libwino — C ABI of the B200 (sm_100a) Winograd 3x3 convolution engine.
 *
 * Drop-in boundary for the convolution hot path of Elon-Wang/cudnnTest.  The reference has no library
 * boundary (every .cuh is #included into one translation unit); the entry points below are what a
 * binding of that path would call.  Each declaration cites the reference interface it replaces
 * (paths relative to the reference repository).
 *
 * Conventions
 *   - plain C types only; every pointer named x, w, u, bias, y, v, m, workspace is a DEVICE pointer
 *     owned by the caller; nothing is allocated or freed by the library unless stated;
 *   - wino_stream_t is a cudaStream_t passed as an opaque pointer (NULL = default stream); all
 *     functions are asynchronous on that stream except wino_wraped_conv, which synchronises like the
 *     reference wrappers do;
 *   - every function returns WINO_OK (0) or a negative WINO_E_* code; wino_last_error_string() gives
 *     the message of the calling thread's last failure;
 *   - 3x3 filters, stride 1, dilation 1, cross-correlation (no kernel flip), zero padding `pad`;
 *   - there is no CPU fallback: without a CUDA device every compute entry point fails with WINO_E_CUDA.
 */
#ifndef WINO_H
#define WINO_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* wino_stream_t;

/* enum class DataLayout {NCHW, NHWC, CHWN}            comparison/DataLayoutTrans.cuh:587-591
 * The filter layout follows the INPUT layout, as in the reference wrappers:
 *   NCHW -> w[k][c][3][3]   (comparison/wrapedConv_NCHW.cuh:869)
 *   NHWC -> w[k][3][3][c]   (comparison/wrapedConv_NHWC.cuh:341)
 *   CHWN -> w[c][3][3][k]   (comparison/wrapedConv_CHWN.cuh:288)                                   */
enum { WINO_NCHW = 0, WINO_NHWC = 1, WINO_CHWN = 2 };

/* storage / arithmetic variants.  FP32: float storage, FP32 FFMA tile GEMM (the reference's
 * arithmetic).  TF32: float storage, tensor-core GEMM on TF32 operands.  BF16: bfloat16 storage,
 * tensor-core GEMM on BF16 or FP16 transform-domain operands.  FP32X3: float storage, tensor-core GEMM in which
 * every transform-domain operand is split into a TF32 head and a TF32 tail (x = hi + lo) and each FP32 product is
 * rebuilt from three TF32 products hi*hi + lo*hi + hi*lo (the dropped lo*lo term is below 2^-22 of the product):
 * FP32-level accuracy (inside the 1e-4 bound of the FP32 variant, not bit-identical to it) at tensor-core speed.
 * Its transformed-filter buffer holds heads and tails, twice the FP32 variant's size (wino_filter_bytes reports it);
 * the scratch has the FP32 variant's size (the input tiles are split inside the tile GEMM).
 * Accumulation is always FP32. */
enum { WINO_FP32 = 0, WINO_TF32 = 1, WINO_BF16 = 2, WINO_FP32X3 = 3 };
enum { WINO_OPERAND_AUTO = 0, WINO_OPERAND_BF16 = 1, WINO_OPERAND_F16 = 2 };
enum { WINO_OUT_SAME = 0, WINO_OUT_FP32 = 1, WINO_OUT_BF16 = 2 };

enum {
    WINO_OK = 0,
    WINO_E_BADARG = -1,
    WINO_E_UNSUPPORTED = -2,
    WINO_E_WORKSPACE = -3,
    WINO_E_CUDA = -4,
    WINO_E_TIMEOUT = -5
};

typedef struct wino_conv_desc {
    int layout_in, layout_out; /* WINO_NCHW / WINO_NHWC / WINO_CHWN; may differ (convLayoutTrans_*) */
    int n, c, h, w, k, pad;    /* batch, input channels, height, width, filters, zero padding        */
    int dtype;                 /* WINO_FP32 / WINO_TF32 / WINO_BF16 / WINO_FP32X3                    */
    int operand;               /* WINO_BF16 only: format of the transformed operands; AUTO = F16 (FP16
                                  operands keep both tile sizes inside the 5e-3 tolerance)          */
    int wino;                  /* output tile size m of F(m x m, 3x3): 2 or 4.  0 = the engine chooses per shape:
                                  F(4x4,3x3), or a direct implicit-GEMM tensor-core kernel where that is faster
                                  (C <= 3; BF16 with C a multiple of 64, TF32 with C a multiple of 32, up to 256
                                  channels, and wider BF16 layers on small images, a handful of images or NCHW tensors; NCHW / CHWN
                                  reach it through NHWC staging in the caller's scratch)                  */
    int relu, has_bias, pool2x2; /* epilogue fused into the output transform: y = pool(relu(conv+b)) */
    int slab_images;           /* images transformed per pass; 0 = as many as fit a 2 GiB scratch       */
    int out_dtype;             /* element type of y: WINO_OUT_SAME (that of x), WINO_OUT_FP32 or WINO_OUT_BF16: the
                                  mixed-precision hand-off between layers, e.g. the last BF16 convolution of a
                                  network writing FP32 NCHW for the FP32 classifier that follows
                                  (netTest/cudnn_test_0124/VGG_Batched/vggCUDNN.cu:173-176 changes layout there).
                                  A y type that differs from x always takes the Winograd pipeline.        */
} wino_conv_desc;

const char* wino_last_error_string(void);
int wino_version(void);

/* Synchronises the current device and reports what the kernels recorded: WINO_OK, WINO_E_TIMEOUT if a
 * bounded device-side wait (mbarrier / tensor-memory hand-off in the tensor-core GEMM) gave up, or
 * WINO_E_CUDA for a CUDA error.  Clears the record.  The reference reports no errors at all (its
 * wrappers return void and leave CUDA errors unchecked, comparison/wrapedConv_NCHW.cuh:482). */
int wino_device_status(void);

/* Bytes of the transformed-filter buffer U (caller allocates).  Replaces the caller-side sizing
 * `36*NSize*KSize` floats, layoutTest/NCHW/convModule_NCHW_padding.cu:44-50. */
size_t wino_filter_bytes(const wino_conv_desc* d);

/* Bytes of scratch wino_conv_forward needs (transformed input V + tile-GEMM output M for one slab of
 * images).  Replaces `36*MSize*KSize` + `36*MSize*NSize` floats, convModule_NCHW_padding.cu:44-50. */
size_t wino_conv_workspace_bytes(const wino_conv_desc* d);

/* U = G g G^T, once per weight tensor.  Replaces wino_kernel_trans_{nchw,nhwc,chwn}_suitFor128
 * (comparison/wrapedConv_NCHW.cuh:861-900, wrapedConv_NHWC.cuh:333-372, wrapedConv_CHWN.cuh:279-319),
 * which the reference re-runs inside every forward call (wrapedConv_NCHW.cuh:423). */
int wino_filter_transform(const wino_conv_desc* d, const void* w, void* u, wino_stream_t stream);

/* y = [pool2x2](relu(conv3x3(x, w) + bias)).  Replaces the body of wrapedConv_NCHW / _NHWC / _CHWN
 * (comparison/wrapedConv_NCHW.cuh:335-492, wrapedConv_NHWC.cuh:24-112, wrapedConv_CHWN.cuh:16-82),
 * the six convLayoutTrans_X_to_Y (comparison/DataLayoutTrans.cuh:9-584) when layout_out differs, and
 * the separate bias / ReLU / pool passes of netTest/cudnn_test_0124/VGG_Batched/Network.h:456-519.
 * `u` comes from wino_filter_transform with a descriptor that may differ in n and slab_images only: its format
 * follows the other fields, never the batch size (transformed filters, filters repacked for a direct kernel, or both
 * where the engine picks the kernel by batch size).
 * bias: K floats (16-byte aligned) or NULL. */
int wino_conv_forward(const wino_conv_desc* d, const void* x, const void* u, const float* bias, void* y,
                      void* workspace, size_t workspace_bytes, wino_stream_t stream);

/* Convolution forward for callers that cannot allocate device memory.  No counterpart in the reference
 * (its drivers cudaMalloc whatever they need, comparison/layoutCompare.cu:120-126).  Same result as
 * wino_conv_forward, but the slab scratch (V and M) is a fixed array of WINO_STATIC_SCRATCH_BYTES that is
 * part of the library image on every GPU that loads it, so the caller passes tensors only and the call
 * performs no cudaMalloc / cudaFree / allocating library routine.  Meant for hosts whose memory pool is
 * frozen after start-up or that run under a foreign allocator or a no-synchronisation rule.
 * The first call on each device resolves the array's device address: make it before any stream capture.
 * A problem whose one-image slab exceeds the array fails with WINO_E_WORKSPACE.  All calls on a device
 * share the array (it keeps the last call's contents; nothing in it has to start at zero): calls that
 * overlap on the GPU race, so keep them on one stream or otherwise serialised. */
#define WINO_STATIC_SCRATCH_BYTES (64u << 20)
size_t wino_static_scratch_bytes(void);
int wino_conv_forward_static(const wino_conv_desc* d, const void* x, const void* u, const float* bias, void* y,
                             wino_stream_t stream);

/* The reference's wrapper signature, C-callable.  Replaces wrapedConv_<L> (comparison/wrapedConv_NCHW.cuh:8,
 * wrapedConv_NHWC.cuh:8, wrapedConv_CHWN.cuh:8), layoutManager (comparison/DataLayoutTrans.cuh:594-651)
 * and convLayoutTrans_<S>_to_<D> (DataLayoutTrans.cuh:9,101,192,309,418,502).  FP32 path, F(4x4,3x3),
 * square images, filter transform on every call, `*chn` set to numOfFilter on return, device
 * synchronised before returning; the three legacy workspaces must have at least the reference's
 * minimum sizes (36*Mp*Kp, 36*Np*Kp, 36*Mp*Np floats; Mp, Np multiples of 128, Kp of 8).  `*output` is
 * written, never reallocated. */
int wino_wraped_conv(int layout_src, int layout_dst, int bat4Conv, int inside, int* chn, int numOfFilter,
                     int padding, float* m1, float* m2, float* inputTran_gpu, float* filterTran_gpu,
                     float* gemmOutput_gpu, float** output);

/* Pure relayout NCHW <-> NHWC <-> CHWN of an (n, c, h, w) tensor; dtype WINO_FP32 (4-byte) or
 * WINO_BF16 (2-byte elements).  The reference has no such kernel (its data was relaid out offline,
 * netTest/cudnn_test_0124/VGG_Batched/vggCUDNN.cu:45-48); this is the standalone converter. */
int wino_layout_convert(int layout_src, int layout_dst, int n, int c, int h, int w, int dtype, const void* in,
                        void* out, wino_stream_t stream);

/* 2x2 stride-2 max-pool in any layout.  Replaces maxPool_CHWN
 * (netTest/cudnn_test_0124/VGG_Batched/CHWN_support.cuh:198-270) and the cudnnPoolingForward call of
 * Network.h:314-366 for block ends that are not fused into the convolution. */
int wino_maxpool2x2(int layout, int n, int c, int h, int w, int dtype, const void* in, void* out,
                    wino_stream_t stream);

/* TEST-ONLY: launches one small CTA in which a bounded device-side wait runs out after `limit_ms` (1 ... 1000)
 * milliseconds, because nothing ever arrives on its mbarrier.  The CTA records the give-up, lets its other warps leave
 * through the abort flag, frees its tensor memory and returns by itself; the next wino_device_status() returns
 * WINO_E_TIMEOUT once, the one after that WINO_OK.  No counterpart in the reference (its kernels have no waits to
 * bound); it exists so that the give-up path of the tensor-core kernels' waits can be exercised without a fault. */
int wino_selftest_wait_timeout(int limit_ms, wino_stream_t stream);

/* ---- measurement hooks ----------------------------------------------------------------------------
 * wino_launch_count: kernels launched by this process through the library so far.
 * wino_profile_enable(1): from now on every kernel launched by wino_conv_forward / wino_filter_transform is
 * bracketed by a pair of CUDA events on its own stream (takes the role of the commented-out five-event
 * per-stage breakdown of comparison/wrapedConv_NCHW.cuh:88-138).  wino_profile_read synchronises the
 * device, adds up the elapsed milliseconds and launches per kernel class since the last read (index 0 input
 * transform, 1 plain tile GEMM (tensor-core or FFMA), 2 output transform, 3 filter transform, 4 row-fused
 * tile GEMM, 5 thin-input (C <= 3) direct convolution, 6 direct tensor-core convolution, 7 unused)
 * and clears the record. */
long long wino_launch_count(void);
int wino_profile_enable(int on);
int wino_profile_read(float stage_ms[8], long long stage_launches[8]);

/* ---- stage-level entry points (tests, profiling) --------------------------------------------------
 * Buffers for a slab of `ns` images starting at image n0 (T = ns*bny*bnx tiles, bny = ceil((h+2p-2)/m)):
 *   V[xi][Tp][Cp]  xi = a*i + j (a = m+2), tile t = (n-n0)*bny*bnx + by*bnx + bx, Cp = c rounded up to
 *                  a multiple of 8, zero filled; element type float (FP32, TF32:
 *                  rounded to TF32) or bf16/f16 per `operand`
 *   U[xi][k][Cp]   same element type as V
 *   M[xi][Tp][Kq]  float, Kq = k rounded up to 8
 * Tp = wino_stage_tile_rows(d, ns) (T rounded up to 128). */
long long wino_stage_tile_rows(const wino_conv_desc* d, int ns);
int wino_stage_cp(const wino_conv_desc* d);
int wino_stage_kq(const wino_conv_desc* d);
/* replaces wino_input_trans_{nchw_suitFor128_2,nhwc_suitFor128,chwn_suitFor128}
 * (wrapedConv_NCHW.cuh:760-856, wrapedConv_NHWC.cuh:266-329, wrapedConv_CHWN.cuh:225-275) */
int wino_stage_input_transform(const wino_conv_desc* d, const void* x, int n0, int ns, void* v,
                               wino_stream_t stream);
/* replaces GEMM_batch_256_128x128_KMKN / _MKNK (comparison/GEMM.cuh:124-255, :4-122) */
int wino_stage_gemm(const wino_conv_desc* d, const void* v, const void* u, float* m, int ns,
                    wino_stream_t stream);
/* replaces wino_invers_{nchw_suitFor128_3,nhwc_suitFor128,chwn_suitFor128_2}
 * (wrapedConv_NCHW.cuh:1034-1114, wrapedConv_NHWC.cuh:376-428, wrapedConv_CHWN.cuh:379-431) */
int wino_stage_output_transform(const wino_conv_desc* d, const float* m, const float* bias, void* y, int n0,
                                int ns, wino_stream_t stream);

/* Row-fused pair used by wino_conv_forward for the tensor-core variants (WINO_TF32, WINO_BF16): the tile
 * GEMM applies the first 1-D output transform in its epilogue and writes
 *   Z[i*m + q][Tp][Kq] = sum_j M[i*a + j] * A[j][q]      (float for WINO_TF32, IEEE half for WINO_BF16)
 * instead of the a*a raw products; the output transform then only applies A^T along i.  Together they
 * replace GEMM_batch_256_128x128_* + wino_invers_* (comparison/GEMM.cuh:124-255,
 * comparison/wrapedConv_NCHW.cuh:1034-1114) with a third (TF32: two thirds) of the product traffic. */
int wino_stage_gemm_rowfused(const wino_conv_desc* d, const void* v, const void* u, void* z, int ns,
                             wino_stream_t stream);
int wino_stage_output_transform_rowfused(const wino_conv_desc* d, const void* z, const float* bias, void* y,
                                         int n0, int ns, wino_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* WINO_H */

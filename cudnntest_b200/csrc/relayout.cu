// Standalone converters: pure relayout NCHW <-> NHWC <-> CHWN and 2x2 max-pool.
//
// The reference has no relayout kernel: its activations and weights were relaid out offline
// (netTest/cudnn_test_0124/VGG_Batched/vggCUDNN.cu:45-48).  All six directions are one batched 2-D
// transpose  in[b][r][q] -> out[b][q][r]  with q contiguous on the input side and r contiguous on the
// output side, done through a 32 x 33 shared-memory tile so both sides move 32 consecutive elements per
// warp.  The pool replaces maxPool_CHWN (netTest/.../VGG_Batched/CHWN_support.cuh:198-270) and the
// cudnnPoolingForward call of Network.h:314-366 where a pool is not fused into the convolution.
// Both are HBM bound: 2 * N*C*H*W elements moved (1.25 * for the pool).
#include "common.cuh"

namespace wino {

template <typename T>
__global__ void __launch_bounds__(256) transpose_batched_kernel(const T* __restrict__ in, T* __restrict__ out, int R, int Q,
                                                                int qtiles, long long sb_in, long long sr_in,
                                                                long long sb_out, long long sq_out) {
    __shared__ T tile[32][33];
    const int qt = blockIdx.x % qtiles;
    const long long b = blockIdx.x / qtiles;
    const int q0 = qt * 32, r0 = blockIdx.y * 32;
    const int lx = threadIdx.x % 32, ly = threadIdx.x / 32;  // 32 x 8
    const T* src = in + b * sb_in;
    T* dst = out + b * sb_out;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ly + 8 * i, q = q0 + lx;
        if (r < R && q < Q) tile[ly + 8 * i][lx] = src[r * sr_in + q];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q = q0 + ly + 8 * i, r = r0 + lx;
        if (r < R && q < Q) dst[q * sq_out + r] = tile[lx][ly + 8 * i];
    }
}

template <typename T>
static int run_transpose(const void* in, void* out, long long B, long long R, long long Q, long long sb_in, long long sr_in,
                         long long sb_out, long long sq_out, cudaStream_t st) {
    if (B == 0 || R == 0 || Q == 0) return WINO_OK;
    const long long qtiles = (Q + 31) / 32, rtiles = (R + 31) / 32;
    if (B * qtiles > 0x7fffffffLL || rtiles > 65535 || R > 0x7fffffffLL || Q > 0x7fffffffLL)
        return fail(WINO_E_UNSUPPORTED, "relayout: tensor too large for one launch");
    dim3 grid((unsigned)(B * qtiles), (unsigned)rtiles);
    count_launch();
    transpose_batched_kernel<T><<<grid, 256, 0, st>>>((const T*)in, (T*)out, (int)R, (int)Q, (int)qtiles, sb_in, sr_in,
                                                       sb_out, sq_out);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

int launch_relayout(int src, int dst, int n, int c, int h, int w, int esize, const void* in, void* out,
                    cudaStream_t st) {
    const long long N = n, C = c, HW = (long long)h * w;
    long long B, R, Q, sbi, sri, sbo, sqo;
    if (src == dst) {
        WINO_CUDA_CHECK(cudaMemcpyAsync(out, in, (size_t)(N * C * HW * esize), cudaMemcpyDeviceToDevice, st));
        return WINO_OK;
    }
    if (src == WINO_NCHW && dst == WINO_NHWC) { B = N; R = C; Q = HW; sbi = C * HW; sri = HW; sbo = HW * C; sqo = C; }
    else if (src == WINO_NHWC && dst == WINO_NCHW) { B = N; R = HW; Q = C; sbi = HW * C; sri = C; sbo = C * HW; sqo = HW; }
    else if (src == WINO_NCHW && dst == WINO_CHWN) { B = 1; R = N; Q = C * HW; sbi = 0; sri = C * HW; sbo = 0; sqo = N; }
    else if (src == WINO_CHWN && dst == WINO_NCHW) { B = 1; R = C * HW; Q = N; sbi = 0; sri = N; sbo = 0; sqo = C * HW; }
    else if (src == WINO_NHWC && dst == WINO_CHWN) { B = HW; R = N; Q = C; sbi = C; sri = HW * C; sbo = N; sqo = HW * N; }
    else if (src == WINO_CHWN && dst == WINO_NHWC) { B = HW; R = C; Q = N; sbi = N; sri = HW * N; sbo = C; sqo = HW * C; }
    else return fail(WINO_E_BADARG, "relayout: bad layout pair %d -> %d", src, dst);
    if (esize == 4) return run_transpose<uint32_t>(in, out, B, R, Q, sbi, sri, sbo, sqo, st);
    if (esize == 2) return run_transpose<uint16_t>(in, out, B, R, Q, sbi, sri, sbo, sqo, st);
    return fail(WINO_E_BADARG, "relayout: element size %d not supported", esize);
}

// 2x2 stride-2 max-pool, one thread per output element, threads ordered along the layout's memory order
template <typename T>
__global__ void __launch_bounds__(256) maxpool_kernel(const T* __restrict__ in, T* __restrict__ out, int layout, int N,
                                                      int C, int H, int W, long long total) {
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total) return;
    const int PH = H / 2, PW = W / 2;
    int n, c, ph, pw;
    long long r = idx;
    if (layout == WINO_NCHW) { pw = r % PW; r /= PW; ph = r % PH; r /= PH; c = r % C; n = (int)(r / C); }
    else if (layout == WINO_NHWC) { c = r % C; r /= C; pw = r % PW; r /= PW; ph = r % PH; n = (int)(r / PH); }
    else { n = r % N; r /= N; pw = r % PW; r /= PW; ph = r % PH; c = (int)(r / PH); }
    const Strides s = act_strides(layout, N, C, H, W);
    const T* p = in + n * s.n + c * s.c + (2 * ph) * s.h + (2 * pw) * s.w;
    const float a = to_float<T>(p[0]), b = to_float<T>(p[s.w]), cc = to_float<T>(p[s.h]), d = to_float<T>(p[s.h + s.w]);
    out[idx] = from_float<T>(fmaxf(fmaxf(a, b), fmaxf(cc, d)));
}

int launch_maxpool(int layout, int n, int c, int h, int w, int dtype, const void* in, void* out, cudaStream_t st) {
    const long long total = (long long)n * c * (h / 2) * (w / 2);
    if (total == 0) return WINO_OK;
    const long long blocks = (total + 255) / 256;
    if (blocks > 0x7fffffffLL) return fail(WINO_E_UNSUPPORTED, "maxpool: tensor too large for one launch");
    count_launch();
    if (dtype == WINO_BF16)
        maxpool_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, layout,
                                                                          n, c, h, w, total);
    else
        maxpool_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)in, (float*)out, layout, n, c, h, w, total);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

}  // namespace wino

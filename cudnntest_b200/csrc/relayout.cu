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

// 2-byte elements, even extents and strides: 64 x 64 element tiles moved as 4-byte words on both sides (a warp reads
// 128 bytes along q and writes 128 bytes along r), the pairing is changed inside shared memory.
__global__ void __launch_bounds__(256) transpose_batched_pairs_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int R,
                                                                      int Q, int qtiles, long long sb_in, long long sr_in,
                                                                      long long sb_out, long long sq_out) {
    __shared__ uint16_t tile[64][66];
    const int qt = blockIdx.x % qtiles;
    const long long b = blockIdx.x / qtiles;
    const int q0 = qt * 64, r0 = blockIdx.y * 64;
    const int lx = threadIdx.x % 32, ly = threadIdx.x / 32;   // 32 x 8
    const uint16_t* src = in + b * sb_in;
    uint16_t* dst = out + b * sb_out;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = r0 + ly + 8 * i, q = q0 + 2 * lx;
        if (r < R && q < Q) {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(src + r * sr_in + q);
            tile[ly + 8 * i][2 * lx] = (uint16_t)(w & 0xffffu);
            tile[ly + 8 * i][2 * lx + 1] = (uint16_t)(w >> 16);
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int q = q0 + ly + 8 * i, r = r0 + 2 * lx;
        if (r < R && q < Q) {
            const uint32_t w = (uint32_t)tile[2 * lx][ly + 8 * i] | ((uint32_t)tile[2 * lx + 1][ly + 8 * i] << 16);
            *reinterpret_cast<uint32_t*>(dst + q * sq_out + r) = w;
        }
    }
}

// 2-byte elements with every extent, stride and pointer a multiple of 16 bytes: 64 x 64 element tiles moved as
// 16-byte vectors on both sides.  The tile sits in shared memory as 64 rows of 32 words whose 16-byte chunks are XOR-ed
// with (row / 8) % 8, which keeps both the row-wise 16-byte stores and the column-wise word reads conflict free;
// a thread reads the word (two q values) of eight consecutive rows and re-pairs the halves into two 16-byte
// vectors of eight r values each.
__global__ void __launch_bounds__(256) transpose_batched_vec_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int R,
                                                                    int Q, int qtiles, long long sb_in, long long sr_in,
                                                                    long long sb_out, long long sq_out) {
    __shared__ __align__(16) uint32_t tile[64][32];
    const int qt = blockIdx.x % qtiles;
    const long long b = blockIdx.x / qtiles;
    const int q0 = qt * 64, r0 = blockIdx.y * 64;
    const int t = threadIdx.x;
    const uint16_t* src = in + b * sb_in;
    uint16_t* dst = out + b * sb_out;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int row = t / 8 + 32 * u, chunk = t % 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r0 + row < R && q0 + 8 * chunk < Q) v = __ldg(reinterpret_cast<const uint4*>(src + (long long)(r0 + row) * sr_in + q0 + 8 * chunk));
        *reinterpret_cast<uint4*>(&tile[row][(chunk ^ ((row >> 3) & 7)) * 4]) = v;
    }
    __syncthreads();
    const int j = t % 8, qp = t / 8;              // r block of eight rows, pair of q values
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = tile[8 * j + i][qp ^ (j << 2)];
    if (r0 + 8 * j < R) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int q = q0 + 2 * qp + e;
            if (q < Q) {
                const uint32_t sel = e ? 0x7632u : 0x5410u;     // high or low halves of a pair of words
                const uint4 v = make_uint4(__byte_perm(w[0], w[1], sel), __byte_perm(w[2], w[3], sel), __byte_perm(w[4], w[5], sel),
                                           __byte_perm(w[6], w[7], sel));
                *reinterpret_cast<uint4*>(dst + (long long)q * sq_out + r0 + 8 * j) = v;
            }
        }
    }
}

// 4-byte elements with every extent, stride and pointer a multiple of 16 bytes: 32 x 32 word tiles moved as 16-byte
// vectors on both sides (a thread loads four consecutive q of one row and stores four consecutive r of one column);
// the tile sits in shared memory with a pitch of 33 words, which keeps both the row-wise writes and the column-wise
// reads conflict free.
__global__ void __launch_bounds__(256) transpose_batched_vec4_kernel(const uint32_t* __restrict__ in, uint32_t* __restrict__ out, int R, int Q,
                                                                     int qtiles, long long sb_in, long long sr_in, long long sb_out,
                                                                     long long sq_out) {
    __shared__ uint32_t tile[32][33];
    const int qt = blockIdx.x % qtiles;
    const long long b = blockIdx.x / qtiles;
    const int q0 = qt * 32, r0 = blockIdx.y * 32;
    const int t = threadIdx.x;
    const uint32_t* src = in + b * sb_in;
    uint32_t* dst = out + b * sb_out;
    {
        const int r = t / 8, c4 = (t % 8) * 4;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r0 + r < R && q0 + c4 < Q) v = __ldg(reinterpret_cast<const uint4*>(src + (long long)(r0 + r) * sr_in + q0 + c4));
        tile[r][c4] = v.x; tile[r][c4 + 1] = v.y; tile[r][c4 + 2] = v.z; tile[r][c4 + 3] = v.w;
    }
    __syncthreads();
    {
        const int q = t / 8, r4 = (t % 8) * 4;
        if (q0 + q < Q && r0 + r4 < R)
            *reinterpret_cast<uint4*>(dst + (long long)(q0 + q) * sq_out + r0 + r4) =
                make_uint4(tile[r4][q], tile[r4 + 1][q], tile[r4 + 2][q], tile[r4 + 3][q]);
    }
}

template <typename T>
static int run_transpose(const void* in, void* out, long long B, long long R, long long Q, long long sb_in, long long sr_in,
                         long long sb_out, long long sq_out, cudaStream_t st) {
    if (B == 0 || R == 0 || Q == 0) return WINO_OK;
    if (sizeof(T) == 2 && ((R | Q | sb_in | sr_in | sb_out | sq_out) & 7) == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        const long long qt = (Q + 63) / 64, rt = (R + 63) / 64;
        if (B * qt <= 0x7fffffffLL && rt <= 65535 && R <= 0x7fffffffLL && Q <= 0x7fffffffLL) {
            dim3 grid((unsigned)(B * qt), (unsigned)rt);
            count_launch();
            transpose_batched_vec_kernel<<<grid, 256, 0, st>>>((const uint16_t*)in, (uint16_t*)out, (int)R, (int)Q, (int)qt, sb_in, sr_in,
                                                                sb_out, sq_out);
            WINO_CUDA_CHECK(cudaGetLastError());
            return WINO_OK;
        }
    }
    if (sizeof(T) == 4 && ((R | Q | sb_in | sr_in | sb_out | sq_out) & 3) == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
        const long long qt = (Q + 31) / 32, rt = (R + 31) / 32;
        if (B * qt <= 0x7fffffffLL && rt <= 65535 && R <= 0x7fffffffLL && Q <= 0x7fffffffLL) {
            dim3 grid((unsigned)(B * qt), (unsigned)rt);
            count_launch();
            transpose_batched_vec4_kernel<<<grid, 256, 0, st>>>((const uint32_t*)in, (uint32_t*)out, (int)R, (int)Q, (int)qt, sb_in, sr_in, sb_out,
                                                                 sq_out);
            WINO_CUDA_CHECK(cudaGetLastError());
            return WINO_OK;
        }
    }
    if (sizeof(T) == 2 && ((R | Q | sb_in | sr_in | sb_out | sq_out) & 1) == 0 && (((uintptr_t)in | (uintptr_t)out) & 3) == 0) {
        const long long qt = (Q + 63) / 64, rt = (R + 63) / 64;
        if (B * qt <= 0x7fffffffLL && rt <= 65535 && R <= 0x7fffffffLL && Q <= 0x7fffffffLL) {
            dim3 grid((unsigned)(B * qt), (unsigned)rt);
            count_launch();
            transpose_batched_pairs_kernel<<<grid, 256, 0, st>>>((const uint16_t*)in, (uint16_t*)out, (int)R, (int)Q, (int)qt, sb_in, sr_in,
                                                                  sb_out, sq_out);
            WINO_CUDA_CHECK(cudaGetLastError());
            return WINO_OK;
        }
    }
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

template <typename T>
__device__ __forceinline__ uint4 max16(uint4 a, uint4 b);
template <>
__device__ __forceinline__ uint4 max16<float>(uint4 a, uint4 b) {
    return make_uint4(__float_as_uint(fmaxf(__uint_as_float(a.x), __uint_as_float(b.x))), __float_as_uint(fmaxf(__uint_as_float(a.y), __uint_as_float(b.y))),
                      __float_as_uint(fmaxf(__uint_as_float(a.z), __uint_as_float(b.z))), __float_as_uint(fmaxf(__uint_as_float(a.w), __uint_as_float(b.w))));
}
template <>
__device__ __forceinline__ uint4 max16<__nv_bfloat16>(uint4 a, uint4 b) {
    uint4 r;
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
    __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) pr[i] = __hmax2(pa[i], pb[i]);
    return r;
}

// Pool for layouts whose innermost dimension is not pooled (NHWC: c, CHWN: n): 16-byte vectors along it.
// The tensor is viewed as [outer][H][W][inner] with inner a multiple of the vector length.
template <typename T>
__global__ void __launch_bounds__(256) maxpool_inner_vec_kernel(const T* __restrict__ in, T* __restrict__ out, int H, int W,
                                                                long long inner_vecs, long long total_vecs) {
    constexpr int VE = 16 / (int)sizeof(T);
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total_vecs) return;
    const int PH = H / 2, PW = W / 2;
    const long long iv = idx % inner_vecs;
    long long r = idx / inner_vecs;
    const int pw = (int)(r % PW); r /= PW;
    const int ph = (int)(r % PH);
    const long long outer = r / PH;
    const long long inner = inner_vecs * VE;
    const T* p = in + ((outer * H + 2 * ph) * W + 2 * pw) * inner + iv * VE;
    const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + inner);
    const uint4 c = *reinterpret_cast<const uint4*>(p + (long long)W * inner), d = *reinterpret_cast<const uint4*>(p + (long long)W * inner + inner);
    *reinterpret_cast<uint4*>(out + idx * VE) = max16<T>(max16<T>(a, b), max16<T>(c, d));
}

// NCHW: the pooled dimension w is the contiguous one.  A thread produces VE adjacent outputs of one row from two
// 16-byte vectors of each of the two input rows (W a multiple of 2*VE keeps every vector aligned).
template <typename T>
__global__ void __launch_bounds__(256) maxpool_nchw_vec_kernel(const T* __restrict__ in, T* __restrict__ out, int H, int W,
                                                               long long total_vecs) {
    constexpr int VE = 16 / (int)sizeof(T);
    const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total_vecs) return;
    const int PH = H / 2, PWV = W / (2 * VE);
    const int pv = (int)(idx % PWV);
    long long r = idx / PWV;
    const int ph = (int)(r % PH);
    const long long plane = r / PH;
    const T* p = in + (plane * H + 2 * ph) * W + (long long)pv * 2 * VE;
    __align__(16) T r0[2 * VE], r1[2 * VE], o[VE];
    *reinterpret_cast<uint4*>(r0) = *reinterpret_cast<const uint4*>(p);
    *reinterpret_cast<uint4*>(r0 + VE) = *reinterpret_cast<const uint4*>(p + VE);
    *reinterpret_cast<uint4*>(r1) = *reinterpret_cast<const uint4*>(p + W);
    *reinterpret_cast<uint4*>(r1 + VE) = *reinterpret_cast<const uint4*>(p + W + VE);
#pragma unroll
    for (int e = 0; e < VE; ++e)
        o[e] = from_float<T>(fmaxf(fmaxf(to_float<T>(r0[2 * e]), to_float<T>(r0[2 * e + 1])), fmaxf(to_float<T>(r1[2 * e]), to_float<T>(r1[2 * e + 1]))));
    *reinterpret_cast<uint4*>(out + (plane * PH + ph) * (W / 2) + (long long)pv * VE) = *reinterpret_cast<const uint4*>(o);
}

int launch_maxpool(int layout, int n, int c, int h, int w, int dtype, const void* in, void* out, cudaStream_t st) {
    const long long total = (long long)n * c * (h / 2) * (w / 2);
    if (total == 0) return WINO_OK;
    {
        // NHWC = [n][H][W][c], CHWN = [c][H][W][n]
        const int es = dtype == WINO_BF16 ? 2 : 4, ve = 16 / es;
        const long long inner = layout == WINO_NHWC ? c : layout == WINO_CHWN ? n : 0;
        if (layout == WINO_NCHW && w % (2 * ve) == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
            const long long vecs = total / ve, blocks = (vecs + 255) / 256;
            if (blocks <= 0x7fffffffLL) {
                count_launch();
                if (dtype == WINO_BF16)
                    maxpool_nchw_vec_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, h, w, vecs);
                else
                    maxpool_nchw_vec_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)in, (float*)out, h, w, vecs);
                WINO_CUDA_CHECK(cudaGetLastError());
                return WINO_OK;
            }
        }
        if (inner > 0 && inner % ve == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
            const long long vecs = total / ve, blocks = (vecs + 255) / 256;
            if (blocks <= 0x7fffffffLL) {
                count_launch();
                if (dtype == WINO_BF16)
                    maxpool_inner_vec_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, h, w, inner / ve, vecs);
                else
                    maxpool_inner_vec_kernel<float><<<(unsigned)blocks, 256, 0, st>>>((const float*)in, (float*)out, h, w, inner / ve, vecs);
                WINO_CUDA_CHECK(cudaGetLastError());
                return WINO_OK;
            }
        }
    }
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

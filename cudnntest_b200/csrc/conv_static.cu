// wino_conv_forward_static: the convolution forward for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run a convolution: an
// inference server whose memory pool has been sized and frozen at start-up, a plugin that runs inside
// someone else's allocator and stream discipline, a real-time loop in which an allocation (an implicit
// device synchronisation) is not acceptable.  wino_conv_forward already takes its scratch from the
// caller; this variant needs no scratch argument at all.  The transformed-input buffer V and the
// tile-GEMM product buffer M of one slab of images live in a fixed array in device global memory that is
// part of the library image itself, so every GPU that loads libwino holds WINO_STATIC_SCRATCH_BYTES of it
// from load until the process exits.
//
// What the caller must know:
//   * the first call on a device looks up the array's device address (cudaGetSymbolAddress, once per
//     device, with that device current).  Make that first call before any stream capture begins;
//   * a problem whose single-image slab (V + M of one image) does not fit the array is rejected with
//     WINO_E_WORKSPACE and a message that states both sizes; larger batches are simply processed in
//     more slabs;
//   * every call on a device shares the one array, and it keeps the previous call's contents.  Nothing in
//     it needs to start at zero (each slab overwrites every element it later reads), but two calls that
//     overlap on the GPU — different streams, or different host threads — race on it.  Serialise them.
//   * no cudaMalloc, cudaFree or allocating library routine is called on this path.
#include <atomic>

#include "common.cuh"

namespace wino {
namespace {

constexpr size_t kStaticScratchBytes = (size_t)WINO_STATIC_SCRATCH_BYTES;

// The scratch itself.  In host code this name is only a handle for the symbol, not a device address:
// host code must go through cudaGetSymbolAddress and pass the result to the kernels.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_scratch_ptr[kMaxDevices];      // zero-initialised (static storage)

// Device address of the scratch array on the current device; looked up once per device.  Two host threads that
// make their first call on a device at the same moment both do the look-up and store the same address.
int static_scratch(void** out) {
    int dev = -1;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(WINO_E_UNSUPPORTED, "static scratch: device index %d out of range", dev);
    void* p = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        WINO_CUDA_CHECK(cudaGetSymbolAddress(&p, g_static_scratch));
        if (p == nullptr) return fail(WINO_E_CUDA, "static scratch: cudaGetSymbolAddress returned a null address");
        g_scratch_ptr[dev].store(p, std::memory_order_release);
    }
    *out = p;
    return WINO_OK;
}

}  // namespace
}  // namespace wino

using namespace wino;

extern "C" {

size_t wino_static_scratch_bytes(void) { return kStaticScratchBytes; }

int wino_conv_forward_static(const wino_conv_desc* d, const void* x, const void* u, const float* bias, void* y,
                             wino_stream_t stream) {
    Geometry g;
    int rc = make_geometry(d, &g);
    if (rc) return rc;
    if (d->n == 0) return WINO_OK;
    if (!x || !u || !y) return fail(WINO_E_BADARG, "conv forward (static scratch): NULL tensor pointer");
    if (d->has_bias && !bias) return fail(WINO_E_BADARG, "conv forward (static scratch): has_bias set but bias is NULL");
    if ((rc = check_device())) return rc;
    if (direct_small_c_applies(*d)) return launch_direct_small_c(*d, g, x, u, bias, y, (cudaStream_t)stream);   // needs no scratch
    if (direct_tc_applies(*d)) return launch_direct_tc(*d, g, x, direct_filters(*d, g, u), bias, y, (cudaStream_t)stream);   // needs no scratch
    // NHWC staging of the whole batch has to fit the array; shapes whose filter buffer holds both forms fall back to
    // the Winograd pipeline (slabs) when it does not
    if (direct_via_nhwc_applies(*d) &&
        !(direct_filter_mode(*d) == 2 && direct_via_nhwc_staging_bytes(*d, g) > kStaticScratchBytes)) {
        const size_t need = direct_via_nhwc_staging_bytes(*d, g);
        if (need > kStaticScratchBytes)
            return fail(WINO_E_WORKSPACE,
                        "conv forward (static scratch): the NHWC staging of this layer needs %zu bytes, the built-in array holds %zu; "
                        "use wino_conv_forward with caller-provided scratch for this size", need, kStaticScratchBytes);
        void* staging = nullptr;
        if ((rc = static_scratch(&staging))) return rc;
        return launch_direct_via_nhwc(*d, g, x, direct_filters(*d, g, u), bias, y, staging, kStaticScratchBytes, (cudaStream_t)stream);
    }

    // largest slab whose V + M (with the same 1 KiB carving as wino_conv_forward) fits the array
    const size_t one = v_bytes(g, tile_rows(g, 1)) + prod_bytes(g, tile_rows(g, 1)) + 1024;
    if (one > kStaticScratchBytes)
        return fail(WINO_E_WORKSPACE,
                    "conv forward (static scratch): one image needs %zu bytes of scratch, the built-in array holds %zu; "
                    "use wino_conv_forward with caller-provided scratch for this size", one, kStaticScratchBytes);
    int ns = d->slab_images > 0 ? d->slab_images : (int)((long long)kStaticScratchBytes / per_image_bytes(g));
    if (ns > d->n) ns = d->n;
    if (ns > 65535) ns = 65535;
    if (ns < 1) ns = 1;
    while (ns > 1 && v_bytes(g, tile_rows(g, ns)) + prod_bytes(g, tile_rows(g, ns)) + 1024 > kStaticScratchBytes) --ns;
    // several slabs: start each on a multiple of 8 images where possible, as wino_conv_forward does, so that the CHWN
    // kernels keep their 16-byte vectors along n (a slab that starts elsewhere is still correct, through scalar accesses)
    if (ns < d->n && ns >= 8 && d->slab_images <= 0) ns -= ns % 8;
    if (v_bytes(g, tile_rows(g, ns)) + prod_bytes(g, tile_rows(g, ns)) + 1024 > kStaticScratchBytes)
        return fail(WINO_E_WORKSPACE, "conv forward (static scratch): a slab of %d image(s) exceeds the built-in %zu bytes", ns,
                    kStaticScratchBytes);

    void* scratch = nullptr;
    if ((rc = static_scratch(&scratch))) return rc;
    const long long tp = tile_rows(g, ns);
    const uintptr_t base = ((uintptr_t)scratch + 1023) & ~(uintptr_t)1023;
    void* v = (void*)base;
    void* prod = (void*)(base + v_bytes(g, tp));
    cudaStream_t st = (cudaStream_t)stream;
    for (int n0 = 0; n0 < d->n; n0 += ns) {
        const int cur = d->n - n0 < ns ? d->n - n0 : ns;
        if ((rc = launch_input_transform(*d, g, x, n0, cur, v, tp, st))) return rc;
        if ((rc = run_conv_gemm(g, v, u, prod, d->k, (long long)cur * g.tiles_img, tp, st))) return rc;
        if ((rc = launch_output_transform(*d, g, prod, g.prod_kind, bias, y, n0, cur, tp, st))) return rc;
    }
    return WINO_OK;
}

}  // extern "C"

// Host-side helpers of the TMA / mbarrier kernels: tensor-map encoding through the driver entry point (no
// link-time dependency on libcuda), SM count, and the device status word of the bounded waits.
#include "ptx.cuh"

namespace wino {

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// 0 = fine, otherwise the code of the first bounded wait that gave up on this device
__device__ int g_wait_status = 0;
constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices] = {nullptr};

}  // namespace

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const unsigned long long* dims,
                      const unsigned long long* strides_bytes, const unsigned* box, bool swizzle_128) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail(WINO_E_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t d[5], s[4];
    cuuint32_t b[5], e[5];
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; e[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) s[i] = strides_bytes[i];
    CUresult r = fn(map, dt, (cuuint32_t)rank, const_cast<void*>(base), d, s, b, e, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle_128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(WINO_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return WINO_OK;
}

int sm_count() {
    static int cached[kMaxDevices] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

int status_word(int** ptr) {
    int dev = -1;
    WINO_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(WINO_E_UNSUPPORTED, "device index %d out of range", dev);
    if (!g_status_ptr[dev]) {
        void* p = nullptr;
        WINO_CUDA_CHECK(cudaGetSymbolAddress(&p, g_wait_status));
        g_status_ptr[dev] = (int*)p;
    }
    *ptr = g_status_ptr[dev];
    return WINO_OK;
}

int read_and_clear_status(int* status) {
    WINO_CUDA_CHECK(cudaDeviceSynchronize());
    int* p = nullptr;
    int rc = status_word(&p);
    if (rc) return rc;
    int s = 0;
    WINO_CUDA_CHECK(cudaMemcpy(&s, p, sizeof(int), cudaMemcpyDeviceToHost));
    if (s != 0) WINO_CUDA_CHECK(cudaMemset(p, 0, sizeof(int)));
    *status = s;
    return WINO_OK;
}

}  // namespace wino

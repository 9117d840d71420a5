// Self-test of the bounded device-side waits: one small CTA with the role structure of the tensor-core kernels
// (a producer warp, a warp that owns tensor memory, two consumer warps) in which the producer waits, with a limit of
// a few milliseconds given by the caller, on an mbarrier that nothing ever arrives on.
//
// What has to happen, and what the GPU test checks through wino_device_status(): the producer's wait gives up after
// the limit, records its code in the device status word and raises the CTA's abort flag; the other warps, parked in
// waits with the normal 2 s limit, see the flag and leave at once; the CTA waits out the drain interval, frees its
// tensor memory and returns by itself.  Nothing faults and nothing waits without a limit, so the context stays
// usable: the next status read is clean.  This is the only way the give-up path of ptx.cuh (mbar_wait_bounded,
// drain_after_abort) runs at all, since the production kernels' waits never time out when they work.
#include "ptx.cuh"
#include "tcgen05.cuh"

namespace wino {

namespace {

constexpr int SELFTEST_WAIT_CODE = 90;

__global__ void __launch_bounds__(128, 1) wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    const uint32_t bar_never = smem_u32(&bars[0]), bar_parked = smem_u32(&bars[1]);
    const int warp = threadIdx.x / 32;
    if (threadIdx.x == 0) {
        mbar_init(bar_never, 1);
        mbar_init(bar_parked, 1);
        abort_word = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), 32);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);

    if (warp == 0) {
        // the producer role: its ring slot never becomes free
        const bool issuer = elect_one();
        const bool ok = mbar_wait_warp(bar_never, 0, abort_flag, status, SELFTEST_WAIT_CODE, limit_ns);
        if (!ok && issuer) drain_after_abort();
    } else {
        // MMA and epilogue roles: parked on a barrier the producer would have completed; they leave through the abort flag
        (void)mbar_wait_warp(bar_parked, 0, abort_flag, status, SELFTEST_WAIT_CODE + 1);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, 32);
    }
}

}  // namespace

}  // namespace wino

using namespace wino;

extern "C" int wino_selftest_wait_timeout(int limit_ms, wino_stream_t stream) {
    if (limit_ms < 1 || limit_ms > 1000) return fail(WINO_E_BADARG, "wait self-test: limit of %d ms outside 1 ... 1000", limit_ms);
    int rc = check_device();
    if (rc) return rc;
    int* status = nullptr;
    if ((rc = status_word(&status))) return rc;
    count_launch();
    wait_timeout_selftest_kernel<<<1, 128, 0, (cudaStream_t)stream>>>(status, (unsigned long long)limit_ms * 1000000ull);
    WINO_CUDA_CHECK(cudaGetLastError());
    return WINO_OK;
}

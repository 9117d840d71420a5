// Thin inline-PTX wrappers shared by the TMA / mbarrier based kernels (sm_100a).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace wino {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // every device-side wait gives up after 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_timer() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// Bounded wait on an mbarrier phase.  Returns false if the CTA is aborting (abort_flag, in shared memory,
// was raised by another thread) or if this wait ran out of time, in which case it raises the flag and
// records `code` in the global status word (first failure wins).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                                  int code, unsigned long long limit_ns = WAIT_LIMIT_NS) {
    unsigned long long t0 = 0;
    for (uint32_t it = 0;; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 0xff) == 0xff) {
            if (*abort_flag) return false;
            const unsigned long long now = global_timer();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit_ns) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
}

// The same wait executed by all 32 lanes of a warp, with one verdict for the warp (so that warp-uniform code can follow).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                               unsigned long long limit_ns = WAIT_LIMIT_NS) {
    const bool ok = mbar_wait_bounded(bar, parity, abort_flag, status, code, limit_ns);
    return __all_sync(0xffffffffu, ok);
}
// One lane of a fully active warp (the same lane every time it is called by that warp).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "elect.sync _|p, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// After an abort: give TMA copies that were already issued time to land before the CTA's shared memory is released.
__device__ __forceinline__ void drain_after_abort() {
    const unsigned long long t0 = global_timer();
    while (global_timer() - t0 < 1000000ull) __nanosleep(1000);
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// ---- programmatic dependent launch -------------------------------------------------------------------
// A kernel launched with the programmatic-serialisation attribute (launch_kernel below) may become resident while the
// kernel before it in the stream is still running.  pdl_wait() blocks until that kernel has completed and its memory
// is visible: every access to tensors (reads of x, writes of y or scratch) comes after it; what comes before it -
// barrier set-up, tensor-memory allocation, descriptor prefetch - overlaps the predecessor's last wave.
// pdl_launch_dependents() tells the scheduler that the next kernel may start becoming resident as this one's CTAs exit.
// Both are no-ops in a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- CTA pairs (cluster of two) -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// whole-cluster barrier (every thread of every CTA of the cluster executes both halves)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on an mbarrier that may live in the other CTA of the cluster (address from mapa_shared).  CTA-scope release
// on purpose: a cluster-scope release makes the arriving warp wait for its earlier global stores (measured as the
// top stall of the epilogue warps); what the waiter consumes here is tensor memory, ordered by the tcgen05 fences.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// TMA loads issued by either CTA of a pair into its OWN shared memory whose completion bytes are counted on an
// mbarrier of the pair's leader CTA (cluster_bar from mapa_shared).  No multicast: each CTA fetches its own box.
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int c0, int c1, int c2,
                                                 int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(cluster_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// ---- host side (tma_host.cu) ---------------------------------------------------------------------------
// Encodes a tiled tensor map.  dims / box are innermost first; strides_bytes has rank-1 entries (dimension 0 is
// dense).  swizzle: 0 = none, 1 (true) = 128-byte swizzle (inner box extent 128 bytes), 2 = 64-byte swizzle (64 bytes).
int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, int rank, const void* base, const unsigned long long* dims,
                      const unsigned long long* strides_bytes, const unsigned* box, int swizzle);
int sm_count();
// true with WINO_PDL=1: kernels that call pdl_wait() are then launched with programmatic stream serialisation
bool pdl_enabled();

// kernel<<<grid, block, smem, st>>>(args...), with the programmatic-serialisation attribute when `pdl` is set.  Only for
// kernels that execute pdl_wait() before their first access to tensors.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Device address of the status word the bounded waits report to (one per device, resolved once).
int status_word(int** ptr);
int read_and_clear_status(int* status);

}  // namespace wino

// Thin inline-PTX wrappers for the sm_100a asynchronous-copy machinery used by the tuned
// kernels: mbarriers, 1-D bulk copies (cp.async.bulk) and tiled TMA loads
// (cp.async.bulk.tensor).  No cluster multicast is used anywhere.
//
// Every wait is bounded in TIME: a waiter that has seen kWaitLimitNs nanoseconds of the
// GPU's global timer go by records a time-out in the device status word and carries on
// (see wait_parity), so a protocol error can never hang the GPU.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <utility>

namespace msd {
namespace tma {

// Device status word (one per device, owned by status.cu): 0 = fine; otherwise the code
// of the first wait that ran out.  Kernels receive its address as an argument; the host
// reads and clears it through msd_device_status().
int *device_status_ptr(int device);  // host; nullptr on failure

constexpr uint64_t kWaitLimitNs = 4000000000ull;  // 4 s: far beyond any legitimate wait (a layer's kernel runs for milliseconds)
constexpr uint64_t kAbortWaitLimitNs = 200000ull;  // once a time-out happened in the block, later waits give up after 0.2 ms (plus one batch of polls)
constexpr uint32_t kParkNs = 5000u;  // longest time one poll of a wait may stay parked by the hardware

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

// Makes mbarrier initialisation visible to the asynchronous proxy before any copy uses it.
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait with a suspend-time hint: the hardware may park the thread for up to `hint_ns`
// nanoseconds, or until the phase completes, instead of returning at once.  A waiting warp (the
// producer between two ring stages, consumers waiting for data) then does not take issue slots
// from the warps it waits for; measured 1 - 2 % on the backward kernels.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t *bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}

// Bounded wait for the phase with the given parity.  `abort_flag` is a shared-memory word
// of the block: once any thread's wait ran out, all later waits in the block use the short
// limit, the block keeps its control flow (so every barrier is still reached) and skips its
// global stores; the host sees the code in the device status word.  The limit is wall time
// on the GPU's nanosecond timer, read only after a first batch of polls has failed.
__device__ __forceinline__ void wait_parity(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code,
                                            uint64_t limit_ns = kWaitLimitNs) {
#pragma unroll 1
    for (int i = 0; i < 16; ++i)
        if (mbar_try_wait_parked(bar, parity, kParkNs)) return;
    const uint64_t t0 = globaltimer_ns();
#pragma unroll 1
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait_parked(bar, parity, kParkNs)) return;
        const uint64_t limit = *abort_flag ? kAbortWaitLimitNs : limit_ns;
        if (globaltimer_ns() - t0 > limit) break;
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
}

// 1-D bulk copy global -> shared; completion is signalled on `bar` as transaction bytes.
// Both addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Tiled TMA loads (no multicast).  Coordinates are innermost first.  The innermost
// coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tensor_g2s_4d(void *dst_smem, const CUtensorMap *map, int c0, int c1, int c2, int c3, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
            smem_u32(dst_smem)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void tensor_g2s_5d(void *dst_smem, const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(
            smem_u32(dst_smem)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation
// attribute may start while the previous kernel of the stream is still draining: everything
// before grid_dependency_wait() (barrier set-up, staging of the layer's weights) overlaps the
// predecessor's tail; nothing the predecessor wrote may be touched before it.
// allow_dependents() tells the scheduler that the NEXT kernel's blocks may be placed as soon
// as resources free up.  Both are no-ops for kernels launched the ordinary way.
//
// The kernels stage their layer's WEIGHTS before the wait, so the attribute is only safe when
// the predecessor in the stream is known not to write them.  The library therefore asks for it
// only between the layer kernels of one msd_block_forward / msd_block_backward call (whose
// first kernel is launched the ordinary way, i.e. after everything enqueued before the call
// has completed); single-op and slab entry points always launch the ordinary way, so a weight
// tensor produced by the kernel just before them (an initialiser, an optimiser step) is seen.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Host, per calling thread: may the next launches overlap their predecessor's tail?
bool overlap_allowed();
void set_overlap_allowed(bool on);
struct OverlapScope {  // off on entry and on exit; the block entry points switch it on after their first launch
    OverlapScope() { set_overlap_allowed(false); }
    ~OverlapScope() { set_overlap_allowed(false); }
};

// Host: launch `kernel` on `s`, with programmatic stream serialisation when the calling thread allows it.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args &&...args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_allowed() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// Named barrier among `count` threads (count a multiple of 32); id 1..15.
__device__ __forceinline__ void named_barrier(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }

}  // namespace tma
}  // namespace msd

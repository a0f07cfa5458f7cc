// msd_conv_relu_backward_k_noalloc: the ReLU weight-gradient op for callers that must not
// allocate device memory.
//
// Who needs it: code that runs where cudaMalloc is off limits or unaffordable — a plugin
// called from inside another framework's memory pool (which owns all device memory and
// hands the plugin only its input and output buffers), a real-time or serving loop whose
// latency budget excludes an allocator call, or a host with a hard memory cap configured
// up front.  The ordinary entry point, msd_conv_relu_backward_k, asks such callers for a
// `workspace` they have no way to provide.
//
// What it does instead: the per-block partial sums of the two-pass gradient reduction go
// into a fixed array that is part of the library image, `g_noalloc_scratch` below.  Every
// GPU that loads the library therefore holds MSD_NOALLOC_SCRATCH_BYTES (4 MiB) of device
// memory until the process exits, whether or not this entry point is ever called.
//
// Consequences the caller must know:
//  * Shapes whose partial sums need more than the fixed array are refused with
//    MSD_ERR_LIMIT (the message states both numbers); nothing is launched.  The need is
//    what msd_workspace_bytes() reports; for float32 and one output channel it is 320
//    blocks x (c_in x taps + 64) floats + 512 bytes, which fits for c_in <= 356 in 2D
//    (9 taps) and c_in <= 118 in 3D (27 taps).
//  * All calls on a device share the one array.  Two calls that may overlap on the GPU
//    (different streams, no ordering between them) race on it; calls on one stream are
//    ordered and therefore safe.
//  * The array keeps whatever the previous call left there.  Nothing has to be cleared:
//    pass one overwrites every partial that pass two reads.  The one exception: a block
//    whose bounded wait ran out skips its store, so after a call that left a non-zero
//    msd_device_status() the gradient may contain leftovers of an earlier call and must
//    be discarded like every other result of that call.
//  * The first call on each device looks up the array's device address (a host-side
//    runtime query, no allocation).  Make that first call outside any stream capture.
//  * No cudaMalloc, cudaFree or allocating library routine is called on this path.
#include <mutex>
#include "common.cuh"

#define MSD_NOALLOC_SCRATCH_BYTES (4u << 20)

// The scratch array.  In host code this name is only a handle for the runtime: it is NOT a
// device address and must never be passed to a kernel.  The address is obtained below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[MSD_NOALLOC_SCRATCH_BYTES];

namespace {

std::mutex g_mu;
void *g_scratch_ptr[64] = {nullptr};

// Device address of the scratch array on `device`, which must be the current device.
int scratch_address(int device, void **out) {
    if (device < 0 || device >= 64) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "noalloc: device ordinal %d out of range", device);
    std::lock_guard<std::mutex> l(g_mu);
    if (!g_scratch_ptr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess) MSD_FAIL(MSD_ERR_CUDA, "noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        if (!p || ((uintptr_t)p & 255)) MSD_FAIL(MSD_ERR_CUDA, "noalloc: scratch array is not 256-byte aligned");
        g_scratch_ptr[device] = p;
    }
    *out = g_scratch_ptr[device];
    return MSD_OK;
}

}  // namespace

extern "C" MSD_API size_t msd_noalloc_scratch_bytes(void) { return MSD_NOALLOC_SCRATCH_BYTES; }

extern "C" MSD_API int msd_conv_relu_backward_k_noalloc(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output,
                                                        const msd_tensor_t *input, void *grad_kernel, int dilation, int device, void *stream) {
    using namespace msd;
    if (!grad_output || !input) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "conv_relu_backward_k_noalloc: tensors must not be null");
    if (grad_output->ndim != 4 && grad_output->ndim != 5)
        MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "conv_relu_backward_k_noalloc: tensors must be 4- or 5-dimensional");
    int64_t voxels = grad_output->size[0];
    for (int k = 2; k < grad_output->ndim; ++k) voxels *= grad_output->size[k];
    const size_t need = msd_workspace_bytes(dtype, grad_output->ndim, voxels, input->size[1], grad_output->size[1]);
    if (need > MSD_NOALLOC_SCRATCH_BYTES)
        MSD_FAIL(MSD_ERR_LIMIT,
                 "conv_relu_backward_k_noalloc: this shape needs %zu bytes of scratch but the built-in array holds %u; "
                 "use msd_conv_relu_backward_k with a caller-provided workspace",
                 need, (unsigned)MSD_NOALLOC_SCRATCH_BYTES);
    void *scratch = nullptr;
    {
        DeviceGuard g(device);
        MSD_CUDA_TRY(g.status);
        int rc = scratch_address(device, &scratch);
        if (rc) return rc;
    }
    return msd_conv_relu_backward_k(dtype, output, grad_output, input, grad_kernel, dilation, scratch, MSD_NOALLOC_SCRATCH_BYTES, device, stream);
}

// The per-device status word that kernels with bounded waits report time-outs into.
#include <mutex>
#include "common.cuh"
#include "tma.cuh"

namespace msd {
namespace tma {

static __device__ int g_device_status_word = 0;

static std::mutex g_mu;
static int *g_ptr[64] = {nullptr};

// Address of the status word on `device` (which must be the current device).  In host code
// the symbol's name is only a handle; the device address comes from cudaGetSymbolAddress.
int *device_status_ptr(int device) {
    if (device < 0 || device >= 64) return nullptr;
    std::lock_guard<std::mutex> l(g_mu);
    if (!g_ptr[device]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status_word) != cudaSuccess) return nullptr;
        g_ptr[device] = (int *)p;
    }
    return g_ptr[device];
}

// One warp waits on a barrier that nobody arrives at; see msd_selftest_wait_timeout.
__global__ void __launch_bounds__(32) wait_timeout_selftest_kernel(int *status, uint64_t limit_ns, int code) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncwarp();
    wait_parity(&bar, 0, &abort_flag, status, code, limit_ns);
}

}  // namespace tma
}  // namespace msd

extern "C" MSD_API int msd_device_status(int device, void *stream, int *status_out) {
    using namespace msd;
    if (!status_out) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_device_status: status_out is null");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    int *p = tma::device_status_ptr(device);
    if (!p) MSD_FAIL(MSD_ERR_CUDA, "msd_device_status: cannot locate the status word");
    cudaStream_t s = (cudaStream_t)stream;
    int v = 0;
    MSD_CUDA_TRY(cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, s));
    MSD_CUDA_TRY(cudaStreamSynchronize(s));
    if (v != 0) MSD_CUDA_TRY(cudaMemsetAsync(p, 0, sizeof(int), s));
    *status_out = v;
    return MSD_OK;
}

extern "C" MSD_API int msd_selftest_wait_timeout(uint64_t limit_ns, int device, void *stream) {
    using namespace msd;
    if (limit_ns < 1000 || limit_ns > 1000000000ull) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_selftest_wait_timeout: limit_ns must lie in [1e3, 1e9]");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    int *p = tma::device_status_ptr(device);
    if (!p) MSD_FAIL(MSD_ERR_CUDA, "msd_selftest_wait_timeout: cannot locate the status word");
    tma::wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(p, limit_ns, MSD_STATUS_SELFTEST_TIMEOUT);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

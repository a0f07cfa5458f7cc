// 3D instantiations of the fused backward kernel (see fast_backward.cuh).
#include "fast_backward3d_hybrid.cuh"

namespace msd {
namespace fast {

template <int TXQ, int J, bool DO_X, bool DO_K>
static int launch3d(const CUtensorMap *m, const BwdParams &p, int grid, size_t smem, cudaStream_t s) {
    auto kern = fused_backward_kernel<3, TXQ, J, DO_X, DO_K>;
    MSD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MSD_CUDA_TRY(tma::launch_pdl(kern, dim3(grid), dim3(bwd_consumer_warps(3) * 32 + 32), smem, s, m[0], m[1], m[2], m[3], p));
    return MSD_OK;
}

// index: [txq16?][mode], mode 0 = x only, 1 = k only, 2 = both
BwdLaunchFn bwd3d_launchers[2][3] = {
    {launch3d<32, 1, true, false>, launch3d<32, 1, false, true>, launch3d<32, 1, true, true>},
    {launch3d<16, 1, true, false>, launch3d<16, 1, false, true>, launch3d<16, 1, true, true>},
};

static int launch3d_split(const CUtensorMap *m, const BwdParams &p, int grid, size_t smem, cudaStream_t s) {
    auto kern = fused_backward_split_kernel<3>;
    MSD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MSD_CUDA_TRY(tma::launch_pdl(kern, dim3(grid), dim3(kSplitThreads), smem, s, m[0], m[1], m[2], m[3], p));
    return MSD_OK;
}
BwdLaunchFn bwd3d_split_launcher = launch3d_split;

// tensor-core variant: maps[0] = activation stages (8 channels x 2 rows x 128), maps[1] = L2 prefetch box of the
// gradient tiles, maps[2] = halo rows of the gradient channel
static int launch3d_hybrid(const CUtensorMap *m, const BwdParams &p, int grid, size_t smem, cudaStream_t s) {
    auto kern = fused_backward3d_hybrid_kernel;
    // the kernel re-divides its registers between its warpgroups; refuse to launch a build whose
    // register pool is smaller than what it will ask for (setmaxnreg.inc would wait forever)
    static int pool_ok = -1;
    if (pool_ok < 0) {
        cudaFuncAttributes fa;
        MSD_CUDA_TRY(cudaFuncGetAttributes(&fa, kern));
        pool_ok = (fa.numRegs * kHybThreads >= kHybRegBudget) ? 1 : 0;
    }
    if (!pool_ok) MSD_FAIL(MSD_ERR_UNSUPPORTED, "tensor-core 3D backward: this build's register allocation does not fit its warpgroup budgets");
    MSD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MSD_CUDA_TRY(tma::launch_pdl(kern, dim3(grid), dim3(kHybThreads), smem, s, m[0], m[1], m[2], p));
    return MSD_OK;
}
BwdLaunchFn bwd3d_hybrid_launcher = launch3d_hybrid;
size_t bwd3d_hybrid_smem(int C, int Dp, int stages) { return hyb_layout(C, Dp, stages).total; }

}  // namespace fast
}  // namespace msd

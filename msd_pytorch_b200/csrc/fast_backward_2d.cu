// 2D instantiations of the fused backward kernel (see fast_backward.cuh).
#include "fast_backward_split.cuh"

namespace msd {
namespace fast {

template <int TXQ, int J, bool DO_X, bool DO_K>
static int launch2d(const CUtensorMap *m, const BwdParams &p, int grid, size_t smem, cudaStream_t s) {
    auto kern = fused_backward_kernel<2, TXQ, J, DO_X, DO_K>;
    MSD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MSD_CUDA_TRY(tma::launch_pdl(kern, dim3(grid), dim3(bwd_consumer_warps(2) * 32 + 32), smem, s, m[0], m[1], m[2], m[3], p));
    return MSD_OK;
}

// index: [txq16?][J-1][mode], mode 0 = x only, 1 = k only, 2 = both
BwdLaunchFn bwd2d_launchers[2][2][3] = {
    {{launch2d<32, 1, true, false>, launch2d<32, 1, false, true>, launch2d<32, 1, true, true>},
     {launch2d<32, 2, true, false>, launch2d<32, 2, false, true>, launch2d<32, 2, true, true>}},
    {{launch2d<16, 1, true, false>, launch2d<16, 1, false, true>, launch2d<16, 1, true, true>},
     {launch2d<16, 2, true, false>, launch2d<16, 2, false, true>, launch2d<16, 2, true, true>}},
};

// role-split kernel (X warps, K warps, builders of the table of M): fast_backward_split.cuh
static int launch2d_split(const CUtensorMap *m, const BwdParams &p, int grid, size_t smem, cudaStream_t s) {
    auto kern = fused_backward_split_kernel<2>;
    MSD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MSD_CUDA_TRY(tma::launch_pdl(kern, dim3(grid), dim3(kSplitThreads), smem, s, m[0], m[1], m[2], m[3], p));
    return MSD_OK;
}
BwdLaunchFn bwd2d_split_launcher = launch2d_split;

}  // namespace fast
}  // namespace msd

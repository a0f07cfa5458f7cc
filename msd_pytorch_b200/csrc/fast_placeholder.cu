#include "kernels.h"
namespace msd { namespace fast {
int num_variants(int) { return 0; }
bool forward_supported(const View &, const View &, int, int) { return false; }
int forward(bool, const View &, const float *, const float *, const View &, int, int, int, cudaStream_t) { return MSD_ERR_UNSUPPORTED; }
bool backward_supported(const BackwardArgs &) { return false; }
size_t backward_workspace_bytes(int, int64_t) { return 0; }
int backward(const BackwardArgs &, int, cudaStream_t) { return MSD_ERR_UNSUPPORTED; }
}}

// Routing of the tuned forward kernels by dimensionality.
#include "kernels.h"

namespace msd {
namespace fast {

bool forward2d_supported(const View &in, const View &out, int d);
int forward2d(bool relu, const View &in, const float *k, const float *bias, const View &out, int d, int device, cudaStream_t s);

int num_variants(int family) {
    switch (family) {
        case FWD2D: return 3;  // lattice rows x column segments per thread
        case BWD2D: return 2;  // 4 / 8 voxels per thread
        default: return 1;
    }
}

bool forward_supported(const View &in, const View &out, int nd, int d) {
    if (nd == 2) return forward2d_supported(in, out, d);
    return false;
}

int forward(bool relu, const View &in, const float *k, const float *bias, const View &out, int nd, int d, int device, cudaStream_t s) {
    if (nd == 2) return forward2d(relu, in, k, bias, out, d, device, s);
    MSD_FAIL(MSD_ERR_UNSUPPORTED, "no tuned forward kernel for this dimensionality");
}

}  // namespace fast
}  // namespace msd

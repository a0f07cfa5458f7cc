// Routing of the tuned forward kernels.
#include "kernels.h"

namespace msd {
namespace fast {

bool forward_nd_supported(const View &in, const View &out, int nd, int d, const void *ws, size_t wsb);
int forward_nd(bool relu, const View &in, const float *k, const float *bias, const View &out, int nd, int d, void *ws, size_t wsb, int device,
               cudaStream_t s);

int num_forward2d_variants();

int num_variants(int family) {
    switch (family) {
        case FWD2D: return num_forward2d_variants();  // lattice rows x column segments x tile width
        case BWD2D: return 2;  // 4 / 8 voxels per thread
        case FWD3D: return 2;  // 4 / 2 column segments per thread
        case BWD3D: return 2;  // unsplit consumers / X warps + K warps
        default: return 1;
    }
}

bool forward_supported(const View &in, const View &out, int nd, int d, const void *ws, size_t wsb) {
    return forward_nd_supported(in, out, nd, d, ws, wsb);
}

int forward(bool relu, const View &in, const float *k, const float *bias, const View &out, int nd, int d, void *ws, size_t wsb, int device,
            cudaStream_t s) {
    return forward_nd(relu, in, k, bias, out, nd, d, ws, wsb, device, s);
}

}  // namespace fast
}  // namespace msd

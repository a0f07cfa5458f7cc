// Internal interfaces between the C ABI (api.cu) and the kernel files.
#pragma once
#include "common.cuh"

namespace msd {

namespace generic {
size_t workspace_bytes(int dtype, int nd, int64_t nvox, int64_t c_in, int64_t c_out);
int forward(int dtype, bool relu, const View &in, const void *k, const void *bias, const View &out, int nd, int d, cudaStream_t s);
int backward_x(int dtype, bool relu, const View *out, const View &gout, const void *k, const View &gin, int nd, int d, cudaStream_t s);
int backward_k(int dtype, bool relu, const View *out, const View &gout, const View &in, void *gk, int nd, int d, void *ws, size_t wsb,
               cudaStream_t s);
int backward_bias(int dtype, bool relu, const View *out, const View &gout, void *gb, void *ws, size_t wsb, cudaStream_t s);
}  // namespace generic

// Tuned float32 kernels for layers that emit ONE channel (the MSD block with
// width 1).  Each `*_supported` predicate is checked by the dispatcher; when it
// says no, the generic kernel runs instead.
namespace fast {

enum Family { FWD2D = 0, BWD2D = 1, FWD3D = 2, BWD3D = 3, NUM_FAMILIES = 4 };

// z-slab window of the calling thread: while set (z1 > z0), the tuned 3D kernels compute
// only the planes [z0, z1) of the tensors they are given and read the planes around them as
// halo.  Used by the slab entry points of the C ABI; cleared again before they return.
void set_z_window(int z0, int z1);
void get_z_window(int Z, int *z0, int *zw);
// Which half of the two-kernel 3D forward the calling thread's next forward() runs: both (the
// z-tap partial sums on the window widened by the dilation, then the z-gather), only the
// partial sums on exactly the window, or only the z-gather of the window.  The slab entry
// point uses the halves so that neighbouring slabs can exchange partial sums in between.
enum ForwardPhase { FWD_BOTH = 0, FWD_SUMS_ONLY = 1, FWD_GATHER_ONLY = 2 };
void set_forward_phase(int phase);
int get_forward_phase();
int num_variants(int family);
int tuning_set(int family, int dilation, int variant);
int tuning_get(int family, int dilation);

// Forward: out = [relu](bias + conv_d(in)), in has C channels, out has 1.
// `ws` is scratch for the 3D forward (three partial-sum volumes); 2D needs none.
size_t forward_workspace_bytes(int nd, int64_t voxels);
bool forward_supported(const View &in, const View &out, int nd, int d, const void *ws, size_t wsb);
int forward(bool relu, const View &in, const float *k, const float *bias, const View &out, int nd, int d, void *ws, size_t wsb, int device,
            cudaStream_t s);

// Deferred second pass of the weight/bias gradient reduction: the fused backward of every
// layer of a block appends one entry, and one table-driven kernel adds all partials at the end.
struct ReduceEntry {
    const float *pk;  // [nparts][nk] partials of the weight gradient, or null
    const float *pb;  // [nparts] partials of the bias gradient, or null
    float *gk;        // accumulated into
    float *gb;        // accumulated into
    int nparts, nk;
    int64_t pitch;    // elements between consecutive partial rows of pk (0: nk)
    int64_t pitch_b;  // elements between consecutive partials of pb (0: 1)
};
struct ReduceList {
    static const int kMax = 64;
    ReduceEntry e[kMax];
    int count;
    size_t ws_used;
};
int flush_reductions(ReduceList *list, cudaStream_t s);

// Fused backward of one layer.  m = gout * gate(out); for every input channel c:
//   gin[c] += conv_d^T(m, k[c])        (if gin)
//   gk[c,:] += <in[c] shifted, m>      (if gk; deterministic two-pass)
//   gb      += sum m                   (if gb)
// `out` may be null (no gate).  `in` may be null when gk is null.
struct BackwardArgs {
    const View *out;   // [N,1,...] ReLU output (gate) or null
    const View *gout;  // [N,1,...]
    const View *in;    // [N,C,...] or null
    const View *gin;   // [N,C,...] or null
    const float *k;    // [1,C,taps] or null (needed when gin)
    float *gk;         // [1,C,taps] accumulated, or null
    float *gb;         // [1] accumulated, or null
    int nd, d;
    void *ws;
    size_t wsb;
    ReduceList *defer;  // null: reduce right after the layer's kernel
    int mask_channel;   // input channel whose updated gradient is stored gated by in[c] > 0; -1: none (needs gk)
};
// In-place gate of one gradient channel: g = (a > 0) ? g : 0 (views must satisfy the tuned
// kernels' alignment rules).
bool gate_channel_supported(const View &g, const View &a);
int gate_channel(const View &g, const View &a, int device, cudaStream_t s);
bool backward_supported(const BackwardArgs &a);
size_t backward_workspace_bytes(int nd, int64_t c_in);
int backward(const BackwardArgs &a, int device, cudaStream_t s);

// Final 1x1 layer over the dense buffer (float32, up to 8 output channels, aligned views).
bool final_supported(const View &res, const View &out);
size_t final_workspace_bytes(int64_t c_in, int64_t c_out);
int final_forward(const View &res, const float *w, const float *bias, const View &out, int device, cudaStream_t s);
int final_backward(const View &res, const View &gout, const float *w, const View &grad, float *gw, float *gb, void *ws, size_t wsb, int device,
                   cudaStream_t s);

}  // namespace fast
}  // namespace msd

// extern "C" entry points of libmsd_b200: argument validation and dispatch between the
// tuned sm_100a kernels (float32, one output channel) and the generic kernels.
#include <atomic>
#include <string.h>
#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace msd {

thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

static std::atomic<int64_t> g_launches{0}, g_fast_launches{0}, g_split_launches{0}, g_mma_launches{0};
void count_launch(bool fast) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (fast) g_fast_launches.fetch_add(1, std::memory_order_relaxed);
}
void count_split_launch() { g_split_launches.fetch_add(1, std::memory_order_relaxed); }
void count_mma_launch() { g_mma_launches.fetch_add(1, std::memory_order_relaxed); }

static bool same_geometry(const View &a, const View &b) { return a.n == b.n && a.z == b.z && a.y == b.y && a.x == b.x; }

static int check_dtype(int dtype) {
    if (dtype != MSD_F32 && dtype != MSD_F64) MSD_FAIL(MSD_ERR_UNSUPPORTED, "dtype %d is not MSD_F32 or MSD_F64", dtype);
    return MSD_OK;
}

// Mirrors checkDilation (msd_custom_convolutions.cpp:39-52).
static int check_dilation(const char *op, const View &v, int nd, int d) {
    if (d <= 0) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: Dilation must be 1 or greater", op);
    if (d > v.y || d > v.x || (nd == 3 && d > v.z)) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: Dilation cannot be greater than size of image.", op);
    return MSD_OK;
}

// Mirrors checkInOutShape (msd_custom_convolutions.cpp:69-83).
static int views2(const char *op, const msd_tensor_t *a, const msd_tensor_t *b, View *va, View *vb, int *nd) {
    if (!make_view(a, va) || !make_view(b, vb)) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: tensors must be 4- or 5-dimensional and non-null", op);
    if (a->ndim != b->ndim) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: tensors differ in number of dimensions", op);
    if (va->n != vb->n) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: Input batch dimension does not match output batch dimension.", op);
    if (!same_geometry(*va, *vb)) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: Input shape does not match output shape.", op);
    *nd = a->ndim - 2;
    return MSD_OK;
}

static int forward_impl(const char *op, bool relu, int dtype, const msd_tensor_t *input, const void *kernel, const void *bias,
                        const msd_tensor_t *output, int d, void *ws, size_t wsb, int device, void *stream) {
    int rc = check_dtype(dtype);
    if (rc) return rc;
    View in, out;
    int nd;
    if ((rc = views2(op, input, output, &in, &out, &nd))) return rc;
    if (!kernel || !bias) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: kernel and bias must not be null", op);
    if ((rc = check_dilation(op, in, nd, d))) return rc;
    if (ws && ((uintptr_t)ws & 255)) MSD_FAIL(MSD_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned", op);
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MSD_F32 && out.c == 1 && fast::forward_supported(in, out, nd, d, ws, wsb))
        return fast::forward(relu, in, (const float *)kernel, (const float *)bias, out, nd, d, ws, wsb, device, s);
    return generic::forward(dtype, relu, in, kernel, bias, out, nd, d, s);
}

static int backward_x_impl(const char *op, bool relu, int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output, const void *kernel,
                           const msd_tensor_t *grad_input, int d, int device, void *stream) {
    int rc = check_dtype(dtype);
    if (rc) return rc;
    View out, gout, gin;
    int nd;
    if ((rc = views2(op, grad_output, grad_input, &gout, &gin, &nd))) return rc;
    if (relu) {
        int nd2;
        if ((rc = views2(op, output, grad_output, &out, &gout, &nd2))) return rc;
        if (out.c != gout.c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: output and grad_output differ in channels", op);
    }
    if (!kernel) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: kernel must not be null", op);
    if ((rc = check_dilation(op, gout, nd, d))) return rc;
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MSD_F32 && gout.c == 1) {
        fast::BackwardArgs a{relu ? &out : nullptr, &gout, nullptr, &gin, (const float *)kernel, nullptr, nullptr, nd, d, nullptr, 0, nullptr, -1};
        if (fast::backward_supported(a)) return fast::backward(a, device, s);
    }
    return generic::backward_x(dtype, relu, relu ? &out : nullptr, gout, kernel, gin, nd, d, s);
}

static int backward_k_impl(const char *op, bool relu, int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output,
                           const msd_tensor_t *input, void *grad_kernel, int d, void *ws, size_t wsb, int device, void *stream) {
    int rc = check_dtype(dtype);
    if (rc) return rc;
    View out, gout, in;
    int nd;
    if ((rc = views2(op, input, grad_output, &in, &gout, &nd))) return rc;
    if (relu) {
        int nd2;
        if ((rc = views2(op, output, grad_output, &out, &gout, &nd2))) return rc;
        if (out.c != gout.c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: output and grad_output differ in channels", op);
    }
    if (!grad_kernel) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: grad_kernel must not be null", op);
    if ((rc = check_dilation(op, in, nd, d))) return rc;
    if (ws && ((uintptr_t)ws & 255)) MSD_FAIL(MSD_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned", op);
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == MSD_F32 && gout.c == 1) {
        fast::BackwardArgs a{relu ? &out : nullptr, &gout, &in, nullptr, nullptr, (float *)grad_kernel, nullptr, nd, d, ws, wsb, nullptr, -1};
        if (fast::backward_supported(a)) return fast::backward(a, device, s);
    }
    return generic::backward_k(dtype, relu, relu ? &out : nullptr, gout, in, grad_kernel, nd, d, ws, wsb, s);
}

static int backward_bias_impl(const char *op, bool relu, int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output, void *grad_bias,
                              void *ws, size_t wsb, int device, void *stream) {
    int rc = check_dtype(dtype);
    if (rc) return rc;
    View out, gout;
    if (!make_view(grad_output, &gout)) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: grad_output must be 4- or 5-dimensional and non-null", op);
    if (relu) {
        int nd2;
        if ((rc = views2(op, output, grad_output, &out, &gout, &nd2))) return rc;
        if (out.c != gout.c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: output and grad_output differ in channels", op);
    }
    if (!grad_bias) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: grad_bias must not be null", op);
    if (ws && ((uintptr_t)ws & 255)) MSD_FAIL(MSD_ERR_WORKSPACE, "%s: workspace must be 256-byte aligned", op);
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    return generic::backward_bias(dtype, relu, relu ? &out : nullptr, gout, grad_bias, ws, wsb, (cudaStream_t)stream);
}

static View channel_slice(const View &v, int64_t c0, int64_t nc, size_t elem) {
    View s = v;
    s.p = (char *)v.p + c0 * v.sc * (int64_t)elem;
    s.c = nc;
    return s;
}

}  // namespace msd

using namespace msd;

extern "C" {

int msd_version(void) { return 100; }

const char *msd_last_error_string(void) { return g_error; }

size_t msd_workspace_bytes(int dtype, int ndim, int64_t voxels, int64_t c_in, int64_t c_out) {
    const int nd = ndim == 5 ? 3 : 2;
    size_t a = generic::workspace_bytes(dtype, nd, voxels, c_in, c_out);
    size_t b = fast::backward_workspace_bytes(nd, c_in);
    return a > b ? a : b;
}

size_t msd_forward_workspace_bytes(int dtype, int ndim, int64_t voxels) {
    return dtype == MSD_F32 ? fast::forward_workspace_bytes(ndim == 5 ? 3 : 2, voxels) : 0;
}

int msd_conv_forward(int dtype, const msd_tensor_t *input, const void *kernel, const void *bias, const msd_tensor_t *output, int dilation,
                     void *workspace, size_t workspace_bytes, int device, void *stream) {
    return forward_impl("conv_forward", false, dtype, input, kernel, bias, output, dilation, workspace, workspace_bytes, device, stream);
}

int msd_conv_relu_forward(int dtype, const msd_tensor_t *input, const void *kernel, const void *bias, const msd_tensor_t *output, int dilation,
                          void *workspace, size_t workspace_bytes, int device, void *stream) {
    return forward_impl("conv_relu_forward", true, dtype, input, kernel, bias, output, dilation, workspace, workspace_bytes, device, stream);
}

int msd_conv_backward_x(int dtype, const msd_tensor_t *grad_output, const void *kernel, const msd_tensor_t *grad_input, int dilation, int device,
                        void *stream) {
    return backward_x_impl("conv_backward_x", false, dtype, nullptr, grad_output, kernel, grad_input, dilation, device, stream);
}

int msd_conv_relu_backward_x(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output, const void *kernel,
                             const msd_tensor_t *grad_input, int dilation, int device, void *stream) {
    return backward_x_impl("conv_relu_backward_x", true, dtype, output, grad_output, kernel, grad_input, dilation, device, stream);
}

int msd_conv_backward_k(int dtype, const msd_tensor_t *grad_output, const msd_tensor_t *input, void *grad_kernel, int dilation, void *workspace,
                        size_t workspace_bytes, int device, void *stream) {
    return backward_k_impl("conv_backward_k", false, dtype, nullptr, grad_output, input, grad_kernel, dilation, workspace, workspace_bytes, device,
                           stream);
}

int msd_conv_relu_backward_k(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output, const msd_tensor_t *input, void *grad_kernel,
                             int dilation, void *workspace, size_t workspace_bytes, int device, void *stream) {
    return backward_k_impl("conv_relu_backward_k", true, dtype, output, grad_output, input, grad_kernel, dilation, workspace, workspace_bytes,
                           device, stream);
}

int msd_conv_backward_bias(int dtype, const msd_tensor_t *grad_output, void *grad_bias, void *workspace, size_t workspace_bytes, int device,
                           void *stream) {
    return backward_bias_impl("conv_backward_bias", false, dtype, nullptr, grad_output, grad_bias, workspace, workspace_bytes, device, stream);
}

int msd_conv_relu_backward_bias(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output, void *grad_bias, void *workspace,
                                size_t workspace_bytes, int device, void *stream) {
    return backward_bias_impl("conv_relu_backward_bias", true, dtype, output, grad_output, grad_bias, workspace, workspace_bytes, device, stream);
}

static int block_checks(const char *op, int dtype, const msd_tensor_t *result, int c_in, int depth, int width, const void *const *weights,
                        const int *dilations, View *r, int *nd) {
    int rc = check_dtype(dtype);
    if (rc) return rc;
    if (!make_view(result, r)) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: buffer must be 4- or 5-dimensional and non-null", op);
    *nd = result->ndim - 2;
    if (c_in < 1 || depth < 1 || width < 1) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: c_in, depth and width must be at least 1", op);
    if (r->c != (int64_t)c_in + (int64_t)depth * width)
        MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: buffer has %lld channels, expected c_in + depth*width = %lld", op, (long long)r->c,
                 (long long)c_in + (long long)depth * width);
    if (!weights || !dilations) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: weights and dilations must not be null", op);
    for (int i = 0; i < depth; ++i) {
        if (!weights[i]) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: weights[%d] is null", op, i);
        if ((rc = check_dilation(op, *r, *nd, dilations[i]))) return rc;
    }
    return MSD_OK;
}

int msd_block_forward(int dtype, const msd_tensor_t *result, int c_in, int depth, int width, const void *const *weights, const void *bias,
                      const int *dilations, void *workspace, size_t workspace_bytes, int device, void *stream) {
    View r;
    int nd;
    int rc = block_checks("msd_block_forward", dtype, result, c_in, depth, width, weights, dilations, &r, &nd);
    if (rc) return rc;
    if (!bias) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_block_forward: bias must not be null");
    if (workspace && ((uintptr_t)workspace & 255)) MSD_FAIL(MSD_ERR_WORKSPACE, "msd_block_forward: workspace must be 256-byte aligned");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t es = dtype == MSD_F64 ? 8 : 4;
    tma::OverlapScope overlap;  // the first kernel is launched the ordinary way, the later layers may overlap their predecessor
    for (int i = 0; i < depth; ++i) {
        const int64_t n_i = c_in + (int64_t)i * width;
        View in = channel_slice(r, 0, n_i, es);
        View out = channel_slice(r, n_i, width, es);
        const void *b = (const char *)bias + (size_t)i * width * es;
        const int d = dilations[i];
        if (dtype == MSD_F32 && width == 1 && fast::forward_supported(in, out, nd, d, workspace, workspace_bytes))
            rc = fast::forward(true, in, (const float *)weights[i], (const float *)b, out, nd, d, workspace, workspace_bytes, device, s);
        else
            rc = generic::forward(dtype, true, in, weights[i], b, out, nd, d, s);
        if (rc) return rc;
        tma::set_overlap_allowed(true);
    }
    return MSD_OK;
}

size_t msd_block_workspace_bytes(int dtype, int ndim, int64_t voxels, int c_in, int depth, int width) {
    // Room for every layer's partial sums, so that all second-pass reductions of a block can
    // run as one kernel at the end (capped; a smaller buffer only makes them run in batches).
    const int64_t n_max = c_in + (int64_t)(depth - 1) * width;
    const size_t one = msd_workspace_bytes(dtype, ndim, voxels, n_max, width);
    size_t all = 0;
    for (int i = 0; i < depth; ++i) all += fast::backward_workspace_bytes(ndim == 5 ? 3 : 2, c_in + (int64_t)i * width);
    const size_t cap = (size_t)256 << 20;
    if (all > cap) all = cap;
    return all > one ? all : one;
}

// What one layer of a block backward will do; decided on the host from shapes, pointers'
// alignment, dilations and the launch table alone, so that it can be checked without a GPU.
struct LayerDecision {
    bool tuned;        // the fused tuned kernel runs (else the three generic kernels)
    bool gate_first;   // topmost layer: its gradient channel is gated in place before the kernel runs
    bool reads_gated;  // the gradient channel arrives already multiplied by the layer's ReLU gate
    bool gates_below;  // the kernel stores the gradient of channel n_i - 1 multiplied by THAT layer's gate
};

namespace {
struct BlockBackwardPlanner {
    int dtype, nd, c_in, depth, width;
    View r, gr;
    const void *const *weights;
    const int *dilations;
    void *const *grad_weights;           // real call: the pointers; plan call: null, see wants_gw
    const unsigned char *wants_gw;       // plan call: per layer, non-zero = weight gradient wanted (null: all wanted)
    bool plan_only;
    void *grad_bias;
    void *workspace;
    size_t workspace_bytes;
    fast::ReduceList *pending;
    size_t es() const { return dtype == MSD_F64 ? 8 : 4; }
    bool fast_dtype() const { return dtype == MSD_F32 && width == 1; }
    void *gk_of(int i) const {
        if (plan_only) return (!wants_gw || wants_gw[i]) ? (void *)(uintptr_t)256 : nullptr;
        return grad_weights ? grad_weights[i] : nullptr;
    }
    fast::BackwardArgs layer_args(int i, View *out, View *gout, View *in, View *gin) const {
        const int64_t n_i = c_in + (int64_t)i * width;
        *out = channel_slice(r, n_i, width, es());
        *in = channel_slice(r, 0, n_i, es());
        *gout = channel_slice(gr, n_i, width, es());
        *gin = channel_slice(gr, 0, n_i, es());
        const float *k = plan_only ? (const float *)(uintptr_t)256 : (const float *)weights[i];
        return fast::BackwardArgs{out, gout, in, gin, k, (float *)gk_of(i), grad_bias ? (float *)grad_bias + i : nullptr, nd, dilations[i],
                                  workspace, workspace_bytes, pending, -1};
    }
    // `gated`: the gradient channel layer i reads is already multiplied by its ReLU gate (done by
    // the kernel of the layer above when it stored that channel).  A layer hands its gradient over
    // gated only when the layer below will run the tuned kernel as well, judged one layer ahead
    // with that layer's own arguments.
    LayerDecision decide(int i, bool gated, fast::BackwardArgs *a, View *out, View *gout, View *in, View *gin) const {
        LayerDecision dec{false, false, gated, false};
        if (!fast_dtype()) {
            *out = channel_slice(r, c_in + (int64_t)i * width, width, es()), *in = channel_slice(r, 0, c_in + (int64_t)i * width, es());
            *gout = channel_slice(gr, c_in + (int64_t)i * width, width, es()), *gin = channel_slice(gr, 0, c_in + (int64_t)i * width, es());
            return dec;
        }
        *a = layer_args(i, out, gout, in, gin);
        // the topmost gradient channel can be gated in place before the first layer runs
        dec.gate_first = !gated && i == depth - 1 && fast::gate_channel_supported(*gout, *out);
        if (gated || dec.gate_first) a->out = nullptr;  // eligibility is judged with the halo buffers this launch will really use
        dec.tuned = fast::backward_supported(*a);
        if (!dec.tuned) {
            dec.gate_first = false;
            return dec;
        }
        if (a->gk != nullptr && i > 0) {
            View o2, go2, in2, gi2;
            fast::BackwardArgs below = layer_args(i - 1, &o2, &go2, &in2, &gi2);
            below.out = nullptr;  // what that layer would be given after a gated hand-over
            dec.gates_below = fast::backward_supported(below);
        }
        a->mask_channel = dec.gates_below ? (int)(c_in + (int64_t)i * width - 1) : -1;
        return dec;
    }
};
}  // namespace

int msd_block_backward(int dtype, const msd_tensor_t *result, const msd_tensor_t *gradients, int c_in, int depth, int width,
                       const void *const *weights, const int *dilations, void *const *grad_weights, void *grad_bias, void *workspace,
                       size_t workspace_bytes, int device, void *stream) {
    View r, gr;
    int nd, nd2;
    int rc = block_checks("msd_block_backward", dtype, result, c_in, depth, width, weights, dilations, &r, &nd);
    if (rc) return rc;
    if ((rc = views2("msd_block_backward", result, gradients, &r, &gr, &nd2))) return rc;
    if (gr.c != r.c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_block_backward: gradients and result differ in channels");
    if (workspace && ((uintptr_t)workspace & 255)) MSD_FAIL(MSD_ERR_WORKSPACE, "msd_block_backward: workspace must be 256-byte aligned");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    cudaStream_t s = (cudaStream_t)stream;
    fast::ReduceList pending;
    pending.count = 0, pending.ws_used = 0;
    const BlockBackwardPlanner P{dtype, nd, c_in, depth, width, r, gr, weights, dilations, grad_weights, nullptr, false, grad_bias, workspace, workspace_bytes, &pending};
    const size_t es = P.es();
    bool gated = false;
    tma::OverlapScope overlap;  // see msd_block_forward
    for (int i = depth - 1; i >= 0; --i) {
        View out, gout, in, gin;
        fast::BackwardArgs a{};
        const LayerDecision dec = P.decide(i, gated, &a, &out, &gout, &in, &gin);
        const int d = dilations[i];
        void *gk = grad_weights ? grad_weights[i] : nullptr;
        void *gb = grad_bias ? (char *)grad_bias + (size_t)i * width * es : nullptr;
        if (dec.tuned) {
            if (dec.gate_first && (rc = fast::gate_channel(gout, out, device, s))) return rc;
            if ((rc = fast::backward(a, device, s))) return rc;
            tma::set_overlap_allowed(true);
            gated = dec.gates_below;
            continue;
        }
        // the generic kernels use the workspace from its start: finish pending reductions first
        if ((rc = fast::flush_reductions(&pending, s))) return rc;
        // A gradient that arrived already gated must not be gated again from `out`; the look-ahead
        // keeps this from happening, the un-gated kernels are the safe answer if it ever does.
        const bool relu = !gated;
        const View *gate = relu ? &out : nullptr;
        if ((rc = generic::backward_x(dtype, relu, gate, gout, weights[i], gin, nd, d, s))) return rc;
        if (gk && (rc = generic::backward_k(dtype, relu, gate, gout, in, gk, nd, d, workspace, workspace_bytes, s))) return rc;
        if (gb && (rc = generic::backward_bias(dtype, relu, gate, gout, gb, workspace, workspace_bytes, s))) return rc;
        tma::set_overlap_allowed(true);
        gated = false;
    }
    return fast::flush_reductions(&pending, s);
}

int msd_block_backward_plan(int dtype, const msd_tensor_t *result, const msd_tensor_t *gradients, int c_in, int depth, int width,
                            const int *dilations, const unsigned char *wants_grad_weight, size_t workspace_bytes, int *codes_out) {
    View r, gr;
    int nd, nd2;
    if (!codes_out) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_block_backward_plan: codes_out is null");
    const void *dummy = (const void *)(uintptr_t)256;
    // block_checks wants a weight pointer per layer; the plan needs none
    const void *stack_ptrs[64];
    const void **ptrs = stack_ptrs;
    if (depth > 64) MSD_FAIL(MSD_ERR_LIMIT, "msd_block_backward_plan: at most 64 layers per query");
    for (int i = 0; i < depth; ++i) ptrs[i] = dummy;
    int rc = block_checks("msd_block_backward_plan", dtype, result, c_in, depth, width, ptrs, dilations, &r, &nd);
    if (rc) return rc;
    if ((rc = views2("msd_block_backward_plan", result, gradients, &r, &gr, &nd2))) return rc;
    if (gr.c != r.c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_block_backward_plan: gradients and result differ in channels");
    const BlockBackwardPlanner P{dtype, nd, c_in, depth, width, r, gr, nullptr, dilations, nullptr, wants_grad_weight, true, (void *)(uintptr_t)256,
                                 (void *)(uintptr_t)256, workspace_bytes, nullptr};
    bool gated = false;
    for (int i = depth - 1; i >= 0; --i) {
        View out, gout, in, gin;
        fast::BackwardArgs a{};
        const LayerDecision dec = P.decide(i, gated, &a, &out, &gout, &in, &gin);
        codes_out[i] = (dec.tuned ? MSD_PLAN_TUNED : 0) | (dec.gate_first ? MSD_PLAN_GATES_TOP_IN_PLACE : 0) |
                       (dec.reads_gated ? MSD_PLAN_READS_GATED : 0) | (dec.tuned && dec.gates_below ? MSD_PLAN_GATES_CHANNEL_BELOW : 0);
        gated = dec.tuned ? dec.gates_below : false;
    }
    return MSD_OK;
}

// One layer of a block on a z-slab: same kernels as the block entry points, restricted to the
// planes [z_begin, z_end) of the local buffer; the planes outside are halo (read only).
static int slab_checks(const char *op, const msd_tensor_t *buffer, int n_in, int dilation, int z_begin, int z_end, View *r) {
    if (!make_view(buffer, r) || buffer->ndim != 5) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: buffer must be 5-dimensional (N, C, Z, Y, X)", op);
    if (n_in < 1 || n_in >= r->c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: n_in = %d must lie in [1, channels)", op, n_in);
    if (z_begin < 0 || z_end > r->z || z_begin >= z_end) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "%s: bad z window [%d, %d) for %lld planes", op, z_begin, z_end, (long long)r->z);
    return check_dilation(op, *r, 3, dilation);
}

int msd_slab_layer_forward(const msd_tensor_t *buffer, int n_in, const void *weight, const void *bias, int dilation, int z_begin, int z_end,
                           int flags, void *workspace, size_t workspace_bytes, int device, void *stream) {
    View r;
    int rc = slab_checks("msd_slab_layer_forward", buffer, n_in, dilation, z_begin, z_end, &r);
    if (rc) return rc;
    if (!weight || !bias) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_slab_layer_forward: weight and bias must not be null");
    if (flags != 0 && flags != MSD_SLAB_FORWARD_SUMS_ONLY && flags != MSD_SLAB_FORWARD_GATHER_ONLY)
        MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_slab_layer_forward: flags must be 0, MSD_SLAB_FORWARD_SUMS_ONLY or MSD_SLAB_FORWARD_GATHER_ONLY");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    View in = channel_slice(r, 0, n_in, 4), out = channel_slice(r, n_in, 1, 4);
    if (!fast::forward_supported(in, out, 3, dilation, workspace, workspace_bytes))
        MSD_FAIL(MSD_ERR_UNSUPPORTED, "msd_slab_layer_forward: shape, alignment, dilation (1..10) or workspace not supported by the tuned 3D kernel");
    fast::set_z_window(z_begin, z_end);
    fast::set_forward_phase(flags == MSD_SLAB_FORWARD_SUMS_ONLY ? fast::FWD_SUMS_ONLY : flags == MSD_SLAB_FORWARD_GATHER_ONLY ? fast::FWD_GATHER_ONLY
                                                                                                                               : fast::FWD_BOTH);
    rc = fast::forward(true, in, (const float *)weight, (const float *)bias, out, 3, dilation, workspace, workspace_bytes, device, (cudaStream_t)stream);
    fast::set_forward_phase(fast::FWD_BOTH);
    fast::set_z_window(0, 0);
    return rc;
}

int msd_slab_layer_backward(const msd_tensor_t *result, const msd_tensor_t *gradients, int n_in, const void *weight, int dilation, int z_begin,
                            int z_end, void *grad_weight, void *grad_bias, int flags, void *workspace, size_t workspace_bytes, int device,
                            void *stream) {
    View r, gr;
    int rc = slab_checks("msd_slab_layer_backward", result, n_in, dilation, z_begin, z_end, &r);
    if (rc) return rc;
    int nd;
    if ((rc = views2("msd_slab_layer_backward", result, gradients, &r, &gr, &nd))) return rc;
    if (gr.c != r.c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_slab_layer_backward: gradients and result differ in channels");
    if (!weight) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_slab_layer_backward: weight must not be null");
    if (workspace && ((uintptr_t)workspace & 255)) MSD_FAIL(MSD_ERR_WORKSPACE, "msd_slab_layer_backward: workspace must be 256-byte aligned");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    View out = channel_slice(r, n_in, 1, 4), in = channel_slice(r, 0, n_in, 4);
    View gout = channel_slice(gr, n_in, 1, 4), gin = channel_slice(gr, 0, n_in, 4);
    const bool gated_in = (flags & MSD_SLAB_GRADIENT_IS_GATED) != 0;
    const bool gate_next = (flags & MSD_SLAB_GATE_CHANNEL_BELOW) != 0 && grad_weight != nullptr && n_in >= 2;
    fast::BackwardArgs a{gated_in ? nullptr : &out, &gout, &in, &gin, (const float *)weight, (float *)grad_weight, (float *)grad_bias, 3, dilation,
                         workspace, workspace_bytes, nullptr, gate_next ? n_in - 1 : -1};
    if ((flags & MSD_SLAB_GATE_CHANNEL_BELOW) && !gate_next)
        MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_slab_layer_backward: MSD_SLAB_GATE_CHANNEL_BELOW needs grad_weight and n_in >= 2");
    if (!fast::backward_supported(a))
        MSD_FAIL(MSD_ERR_UNSUPPORTED, "msd_slab_layer_backward: shape, alignment, dilation or workspace not supported by the tuned 3D kernel");
    fast::set_z_window(z_begin, z_end);
    rc = fast::backward(a, device, (cudaStream_t)stream);
    fast::set_z_window(0, 0);
    return rc;
}

size_t msd_final_workspace_bytes(int64_t c_in, int64_t c_out) { return fast::final_workspace_bytes(c_in, c_out); }

int msd_final_forward(int dtype, const msd_tensor_t *result, const void *weight, const void *bias, const msd_tensor_t *output, int device,
                      void *stream) {
    View r, o;
    int nd;
    int rc = views2("msd_final_forward", result, output, &r, &o, &nd);
    if (rc) return rc;
    if (!weight || !bias) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_final_forward: weight and bias must not be null");
    if (dtype != MSD_F32 || !fast::final_supported(r, o))
        MSD_FAIL(MSD_ERR_UNSUPPORTED, "msd_final_forward: needs float32, at most 8 output channels, unit x-stride and 16-byte aligned rows");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    return fast::final_forward(r, (const float *)weight, (const float *)bias, o, device, (cudaStream_t)stream);
}

int msd_final_backward(int dtype, const msd_tensor_t *result, const msd_tensor_t *grad_output, const void *weight, const msd_tensor_t *gradients,
                       void *grad_weight, void *grad_bias, void *workspace, size_t workspace_bytes, int device, void *stream) {
    View r, go, gr;
    int nd;
    int rc = views2("msd_final_backward", result, grad_output, &r, &go, &nd);
    if (rc) return rc;
    if ((rc = views2("msd_final_backward", result, gradients, &r, &gr, &nd))) return rc;
    if (gr.c != r.c) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_final_backward: gradients and result differ in channels");
    if (!weight) MSD_FAIL(MSD_ERR_BAD_ARGUMENT, "msd_final_backward: weight must not be null");
    if (workspace && ((uintptr_t)workspace & 255)) MSD_FAIL(MSD_ERR_WORKSPACE, "msd_final_backward: workspace must be 256-byte aligned");
    if (dtype != MSD_F32 || !fast::final_supported(r, go) || !fast::final_supported(gr, go))
        MSD_FAIL(MSD_ERR_UNSUPPORTED, "msd_final_backward: needs float32, at most 8 output channels, unit x-stride and 16-byte aligned rows");
    DeviceGuard g(device);
    MSD_CUDA_TRY(g.status);
    return fast::final_backward(r, go, (const float *)weight, gr, (float *)grad_weight, (float *)grad_bias, workspace, workspace_bytes, device,
                                (cudaStream_t)stream);
}

int msd_tuning_num_variants(int family) { return fast::num_variants(family); }
int msd_tuning_set(int family, int dilation, int variant) { return fast::tuning_set(family, dilation, variant); }
int msd_tuning_get(int family, int dilation) { return fast::tuning_get(family, dilation); }

int64_t msd_launch_count(void) { return g_launches.load(); }
int64_t msd_fast_launch_count(void) { return g_fast_launches.load(); }
int64_t msd_split_launch_count(void) { return g_split_launches.load(); }
int64_t msd_mma_launch_count(void) { return g_mma_launches.load(); }
void msd_reset_launch_count(void) {
    g_launches.store(0);
    g_fast_launches.store(0);
    g_split_launches.store(0);
    g_mma_launches.store(0);
}

}  // extern "C"

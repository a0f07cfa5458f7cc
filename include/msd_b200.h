/*
 * msd_b200 — C ABI of the B200-native Mixed-Scale Dense (MSD) convolution library.
 *
 * Every entry point replaces one function of the reference's native module
 * `msd_custom_convolutions` (ahendriksen/msd_pytorch,
 * msd_pytorch/msd_custom_convolutions.cpp:343-369, launchers declared in
 * msd_pytorch/msd_custom_convolutions/torch_cuda_dispatch.h:4-49) or the Python
 * loop of `MSDBlockFunction` above it (msd_pytorch/msd_block.py:8-134).
 *
 * Conventions
 *  - All pointers are DEVICE pointers owned by the caller; nothing is retained.
 *  - Data tensors are described by `msd_tensor_t`: dimensions in the order
 *    N, C, [Z,] Y, X (ndim 4 = 2D images, ndim 5 = 3D volumes), sizes and
 *    strides in ELEMENTS.  Arbitrary strides are honoured (channel-slice views
 *    of one dense buffer are the normal case).  Convolution weights are dense
 *    `[c_out, c_in, 3, 3(, 3)]`; bias is dense `[c_out]`.
 *  - `dtype` is MSD_F32 or MSD_F64 for every tensor of a call.
 *  - Work is enqueued asynchronously on `stream` (a `cudaStream_t`) of CUDA
 *    device ordinal `device`; the library switches to that device for the call
 *    and restores the previous one.
 *  - Padding is the reference's edge-inclusive reflection: index -k reads k-1,
 *    index n-1+k reads n-k (msd_custom_convolutions/kernel_utils.cuh:30-38);
 *    it requires 1 <= dilation <= every spatial size.
 *  - `grad_input`, `grad_kernel`, `grad_bias` are ACCUMULATED INTO, like the
 *    reference (conv2d_backward_x.cu:103, conv2d_backward_k.cu:52,
 *    conv2d_backward_bias.cu:46); `output` is overwritten.
 *  - Weight and bias gradients are deterministic: per-block partial sums are
 *    written to `workspace` and added in a fixed order by a second kernel.
 *    `workspace` must hold `msd_workspace_bytes()` bytes, be 256-byte aligned
 *    and not be shared by calls that may overlap on the GPU.
 *  - Return value: MSD_OK or an error code; `msd_last_error_string()` gives the
 *    message of the calling thread's last failure.  Nothing throws.
 *  - Thread-safe and re-entrant (the only global state is a mutex-protected
 *    cache of TMA descriptors and launch configurations).
 */
#ifndef MSD_B200_H
#define MSD_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define MSD_API __attribute__((visibility("default")))
#else
#define MSD_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define MSD_OK 0
#define MSD_ERR_BAD_ARGUMENT 1 /* shapes / ranks / dilation do not satisfy the op's contract */
#define MSD_ERR_UNSUPPORTED 2  /* dtype or size outside what the library implements */
#define MSD_ERR_WORKSPACE 3    /* workspace missing, misaligned or too small */
#define MSD_ERR_CUDA 4         /* a CUDA runtime / driver call or a launch failed */
#define MSD_ERR_LIMIT 5        /* size beyond a stated fixed maximum (no-allocation entry point) */

#define MSD_F32 0
#define MSD_F64 1

#define MSD_MAX_DIMS 5

typedef struct msd_tensor {
    void *data;
    int32_t ndim; /* 4 (N,C,Y,X) or 5 (N,C,Z,Y,X) */
    int32_t reserved;
    int64_t size[MSD_MAX_DIMS];
    int64_t stride[MSD_MAX_DIMS]; /* in elements */
} msd_tensor_t;

/* Library version (major*10000 + minor*100 + patch). */
MSD_API int msd_version(void);

/* Message of the calling thread's most recent error ("" if none). */
MSD_API const char *msd_last_error_string(void);

/* Upper bound, in bytes, of the scratch `workspace` any backward entry point
 * below needs for these sizes (`voxels` = N * prod(spatial)). */
MSD_API size_t msd_workspace_bytes(int dtype, int ndim, int64_t voxels, int64_t c_in, int64_t c_out);

/* ---- single operations: the eight functions of `msd_custom_convolutions` ---- */

/* Scratch bytes the forward entry points want for these sizes (0 for 2D and for float64).
 * The tuned 3D forward keeps three partial-sum volumes there; without a workspace
 * (NULL / too small) 3D calls still work but run the generic kernel. */
MSD_API size_t msd_forward_workspace_bytes(int dtype, int ndim, int64_t voxels);

/* conv_forward (msd_custom_convolutions.cpp:85-116; conv2d_forward.cu:22-93, conv3d_forward.cu:22-108) */
MSD_API int msd_conv_forward(int dtype, const msd_tensor_t *input, const void *kernel, const void *bias,
                     const msd_tensor_t *output, int dilation, void *workspace, size_t workspace_bytes,
                     int device, void *stream);

/* conv_relu_forward (msd_custom_convolutions.cpp:213-245; conv2d_forward.cu:95-174, conv3d_forward.cu:110-196) */
MSD_API int msd_conv_relu_forward(int dtype, const msd_tensor_t *input, const void *kernel, const void *bias,
                          const msd_tensor_t *output, int dilation, void *workspace, size_t workspace_bytes,
                          int device, void *stream);

/* conv_backward_x (msd_custom_convolutions.cpp:118-148; conv2d_backward_x.cu:13-106, conv3d_backward_x.cu:13-123) */
MSD_API int msd_conv_backward_x(int dtype, const msd_tensor_t *grad_output, const void *kernel,
                        const msd_tensor_t *grad_input, int dilation, int device, void *stream);

/* conv_relu_backward_x (msd_custom_convolutions.cpp:247-281; conv2d_backward_x.cu:109-208, conv3d_backward_x.cu:125-241) */
MSD_API int msd_conv_relu_backward_x(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output,
                             const void *kernel, const msd_tensor_t *grad_input, int dilation,
                             int device, void *stream);

/* conv_backward_k (msd_custom_convolutions.cpp:150-178; conv2d_backward_k.cu:12-59, conv3d_backward_k.cu:11-64) */
MSD_API int msd_conv_backward_k(int dtype, const msd_tensor_t *grad_output, const msd_tensor_t *input,
                        void *grad_kernel, int dilation, void *workspace, size_t workspace_bytes,
                        int device, void *stream);

/* conv_relu_backward_k (msd_custom_convolutions.cpp:283-316; conv2d_backward_k.cu:61-112, conv3d_backward_k.cu:66-122) */
MSD_API int msd_conv_relu_backward_k(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output,
                             const msd_tensor_t *input, void *grad_kernel, int dilation,
                             void *workspace, size_t workspace_bytes, int device, void *stream);

/* conv_backward_bias (msd_custom_convolutions.cpp:180-211, an ATen sum in the reference) */
MSD_API int msd_conv_backward_bias(int dtype, const msd_tensor_t *grad_output, void *grad_bias,
                           void *workspace, size_t workspace_bytes, int device, void *stream);

/* conv_relu_backward_bias (msd_custom_convolutions.cpp:318-338; conv2d_backward_bias.cu:12-49, conv3d_backward_bias.cu:12-51) */
MSD_API int msd_conv_relu_backward_bias(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output,
                                void *grad_bias, void *workspace, size_t workspace_bytes,
                                int device, void *stream);

/* ---- whole dense block: the loops of MSDBlockFunction (msd_block.py:8-134) ---- */

/* Forward of all `depth` layers over ONE buffer `result[N, c_in + depth*width, ...]`
 * whose first `c_in` channels already hold the input (msd_block.py:30-58).
 * Layer i reads channels [0, c_in + i*width) and writes the next `width` channels:
 * ReLU(conv_{dilations[i]} + bias).  `weights` is a HOST array of `depth` device
 * pointers, weights[i] dense [width, c_in + i*width, 3, 3(, 3)]; `bias` is a device
 * pointer to depth*width values; `dilations` is a HOST array.  `workspace` as for
 * msd_conv_relu_forward (msd_forward_workspace_bytes). */
MSD_API int msd_block_forward(int dtype, const msd_tensor_t *result, int c_in, int depth, int width,
                      const void *const *weights, const void *bias, const int *dilations,
                      void *workspace, size_t workspace_bytes, int device, void *stream);

/* Backward of all layers, last to first (msd_block.py:64-134).  `gradients` has the
 * shape of `result` and holds the gradient w.r.t. every channel on entry; it is
 * updated in place and its first `c_in` channels are the input gradient on return.
 * Higher channels are left in a library-defined state.
 * `grad_weights` is a HOST array of `depth` device pointers (an entry may be NULL to
 * skip that layer's weight gradient); `grad_bias` may be NULL.  Both are accumulated
 * into. */
MSD_API int msd_block_backward(int dtype, const msd_tensor_t *result, const msd_tensor_t *gradients,
                       int c_in, int depth, int width, const void *const *weights,
                       const int *dilations, void *const *grad_weights, void *grad_bias,
                       void *workspace, size_t workspace_bytes, int device, void *stream);

/* Scratch bytes `msd_block_backward` needs. */
MSD_API size_t msd_block_workspace_bytes(int dtype, int ndim, int64_t voxels, int c_in, int depth, int width);

/* ---- final 1x1 layer over the dense buffer ---- */

/* output[n,o,...] = bias[o] + sum_c weight[o,c] * result[n,c,...]: the final layer of the
 * MSD module (MSDFinalLayer, msd_pytorch/msd_module.py:60-88, a Conv1d on the flattened
 * buffer in the reference).  float32, at most 8 output channels, unit x-stride and
 * 16-byte aligned rows; anything else returns MSD_ERR_UNSUPPORTED (the Python layer then
 * uses a library matrix product). */
MSD_API int msd_final_forward(int dtype, const msd_tensor_t *result, const void *weight, const void *bias,
                      const msd_tensor_t *output, int device, void *stream);

/* Backward of the final layer, fused with the set-up of the block backward: WRITES
 * gradients[n,c,...] = sum_o weight[o,c] * grad_output[n,o,...] for every channel of the
 * dense gradient buffer (which msd_block_backward then updates in place - the reference's
 * intermediate gradient tensor and its clone, msd_block.py:83, do not exist here) and
 * accumulates grad_weight[o,c] and grad_bias[o] (either may be NULL) deterministically.
 * `workspace`: msd_final_workspace_bytes(). */
MSD_API int msd_final_backward(int dtype, const msd_tensor_t *result, const msd_tensor_t *grad_output,
                       const void *weight, const msd_tensor_t *gradients, void *grad_weight, void *grad_bias,
                       void *workspace, size_t workspace_bytes, int device, void *stream);
MSD_API size_t msd_final_workspace_bytes(int64_t c_in, int64_t c_out);

/* No counterpart in the reference: what msd_block_backward WOULD do, layer by layer, decided
 * on the host alone (no GPU is touched, data pointers are only inspected for alignment).
 * `codes_out[i]` (i = layer, `depth` <= 64 entries) is a combination of
 *   MSD_PLAN_TUNED                the fused tuned kernel runs (otherwise the generic kernels)
 *   MSD_PLAN_GATES_TOP_IN_PLACE   topmost layer: its gradient channel is gated in place first
 *   MSD_PLAN_READS_GATED          the layer receives its gradient channel already gated
 *   MSD_PLAN_GATES_CHANNEL_BELOW  the layer stores the gradient of the channel below gated
 * A layer gates the channel below only when the layer below runs a tuned kernel too; a gated
 * gradient never meets a kernel that would gate it again.  `wants_grad_weight` (per layer,
 * NULL = all) says for which layers a weight gradient is requested. */
#define MSD_PLAN_TUNED 1
#define MSD_PLAN_GATES_TOP_IN_PLACE 2
#define MSD_PLAN_READS_GATED 4
#define MSD_PLAN_GATES_CHANNEL_BELOW 8
MSD_API int msd_block_backward_plan(int dtype, const msd_tensor_t *result, const msd_tensor_t *gradients, int c_in,
                            int depth, int width, const int *dilations, const unsigned char *wants_grad_weight,
                            size_t workspace_bytes, int *codes_out);

/* ---- z-slab decomposition of one 3D volume over several GPUs ---- */

/* No counterpart in the reference (it has no spatial decomposition).  One layer of the
 * block on a z-slab: `buffer[N, C, Zl, Y, X]` (float32) is this GPU's part of the dense
 * buffer, its planes [z_begin, z_end) owned, the planes below/above them halo copies of
 * the neighbours' planes (at least `dilation` of them, except at the volume's real ends,
 * where the buffer ends too and the edge-inclusive reflection applies).  Writes channel
 * n_in on the owned planes only.  Needs the workspace of msd_forward_workspace_bytes() for
 * the whole local buffer: it holds the three z-tap partial sums u[3][N][Zl][Y][X]
 * (u_t[z] = the in-plane 3x3 sum of plane z with the weights of z-tap t), from which
 * out[z] = relu(bias + u_0[z - d] + u_1[z] + u_2[z + d]).
 * `flags` = 0: both steps in one call; the partial sums are computed on the window widened
 * by `dilation` planes, which reads channels [0, n_in) on halo planes (the caller has
 * exchanged them) and repeats work of the neighbours.
 * `flags` = MSD_SLAB_FORWARD_SUMS_ONLY: only the partial sums, on exactly [z_begin, z_end)
 * (any sub-window of the owned planes; no halo plane of the input is read).
 * `flags` = MSD_SLAB_FORWARD_GATHER_ONLY: only the second step on [z_begin, z_end); the
 * caller has filled u_0 on the `dilation` planes below the owned ones and u_2 on the
 * `dilation` planes above them with the neighbours' partial sums (planes of the same
 * global index), so no layer ever needs an activation halo. */
#define MSD_SLAB_FORWARD_SUMS_ONLY 1
#define MSD_SLAB_FORWARD_GATHER_ONLY 2
MSD_API int msd_slab_layer_forward(const msd_tensor_t *buffer, int n_in, const void *weight, const void *bias,
                           int dilation, int z_begin, int z_end, int flags, void *workspace,
                           size_t workspace_bytes, int device, void *stream);

/* Backward of the same layer on the slab: uses channel n_in of `result` (gate) and of
 * `gradients` on owned + halo planes (the caller has exchanged the gradient halo), adds the
 * input gradient into channels [0, n_in) of `gradients` on the owned planes, and this
 * slab's share of the weight / bias gradient into grad_weight / grad_bias (either may be
 * NULL); the caller sums those over the GPUs.
 * `flags`: MSD_SLAB_GRADIENT_IS_GATED - channel n_in of `gradients` already holds the
 * gradient multiplied by the ReLU gate (result > 0), so no halo of `result` is read;
 * MSD_SLAB_GATE_CHANNEL_BELOW - store the updated gradient of channel n_in - 1 already
 * multiplied by ITS gate (result[n_in - 1] > 0), ready for the next call (needs grad_weight).
 * Chaining the two halves the halo traffic and shared memory of every layer but the top one. */
#define MSD_SLAB_GRADIENT_IS_GATED 1
#define MSD_SLAB_GATE_CHANNEL_BELOW 2
MSD_API int msd_slab_layer_backward(const msd_tensor_t *result, const msd_tensor_t *gradients, int n_in,
                            const void *weight, int dilation, int z_begin, int z_end, void *grad_weight,
                            void *grad_bias, int flags, void *workspace, size_t workspace_bytes, int device,
                            void *stream);

/* ---- launch autotuner (replaces benchmarks/benchmark_block_sizes.py) ---- */

/* Number of launch variants the library has for a kernel family
 * (family: 0 = 2D forward, 1 = 2D backward, 2 = 3D forward, 3 = 3D backward).
 * 3D backward: variant 0 = one kind of consumer warp computes both gradients,
 * variant 1 (default) = warps split by role (input-gradient warps, weight-gradient
 * warps, table builders) for layers with 8 (dilation <= 5) or 10 and more input
 * channels whose x extent is a multiple of 128; variant 2 = the input gradient as a
 * TF32 tensor-core contraction with error-compensated operand splitting (tcgen05,
 * float32-level accuracy), the weight gradient on the CUDA cores (8 to ~88 input
 * channels, x extent a multiple of 128, already gated gradient).
 * 2D backward: variant 0 / 1 (default) = 4 / 8 voxels per thread, one kind of consumer
 * warp; variant 2 = warps split by role as in 3D (x extent a multiple of 128).
 * Forward: tile shapes (rows of the row lattice, column segments per thread, tile
 * width); an untuned 2D forward uses the shapes that won on a large image. */
MSD_API int msd_tuning_num_variants(int family);

/* Force variant `variant` (or -1 = library default) for (family, dilation).
 * Used by the Python autotuner, which times the variants on the caller's shapes
 * and stores the winners on disk. */
MSD_API int msd_tuning_set(int family, int dilation, int variant);
MSD_API int msd_tuning_get(int family, int dilation);

/* Counters for tests and benchmarks: number of kernels this library launched in
 * the calling process since load / since the last reset, and how many of those
 * took the tuned sm_100a path (TMA-staged forward, register-resident fused
 * backward) rather than the generic one. */
MSD_API int64_t msd_launch_count(void);
MSD_API int64_t msd_fast_launch_count(void);
MSD_API int64_t msd_split_launch_count(void); /* of those, launches of the role-split 3D backward kernel */
MSD_API int64_t msd_mma_launch_count(void);   /* of those, launches of the tensor-core 3D backward kernel */
MSD_API void msd_reset_launch_count(void);

/* No counterpart in the reference: msd_conv_relu_backward_k for callers that cannot
 * allocate device memory (a plugin inside another framework's memory pool, a latency-bound
 * serving loop, a host with a fixed memory plan).  It takes no workspace: the partial sums
 * live in a 4 MiB array built into the library, which every GPU that loads the library
 * holds until exit.  Shapes that need more return MSD_ERR_LIMIT and launch nothing (for
 * one output channel: more than 356 input channels in 2D, more than 118 in 3D).  All
 * calls on a device share the array, so calls that may overlap on the GPU race; calls on
 * one stream are safe.  The first call on each device resolves the array's address and
 * should be made outside any stream capture.  Allocates nothing. */
MSD_API int msd_conv_relu_backward_k_noalloc(int dtype, const msd_tensor_t *output, const msd_tensor_t *grad_output,
                                             const msd_tensor_t *input, void *grad_kernel, int dilation,
                                             int device, void *stream);

/* Size in bytes of the built-in scratch array used by msd_conv_relu_backward_k_noalloc. */
MSD_API size_t msd_noalloc_scratch_bytes(void);

/* Waits for `stream`, then reports (and clears) the device status word: 0 when every
 * kernel's internal waits completed, otherwise the code of the first bounded wait that
 * ran out (the affected call's results are then invalid).  The tuned kernels never spin
 * without a limit, so a protocol error shows up here instead of as a hung GPU. */
MSD_API int msd_device_status(int device, void *stream, int *status_out);

/* No counterpart in the reference: self-test of the bounded-wait machinery.  Launches one
 * small block that waits on an mbarrier nobody ever arrives at, with a time limit of
 * `limit_ns` nanoseconds (1000 .. 10^9) on the GPU's timer.  The wait runs out by itself,
 * the kernel returns normally and leaves MSD_STATUS_SELFTEST_TIMEOUT in the device status
 * word, which msd_device_status() then reports and clears.  Nothing traps, faults or
 * spins without a limit; the context stays usable. */
#define MSD_STATUS_SELFTEST_TIMEOUT 99
MSD_API int msd_selftest_wait_timeout(uint64_t limit_ns, int device, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* MSD_B200_H */

// The final 1x1 layer of the MSD module, fused with the dense block's buffers.
//
// In the reference the final layer is a Conv1d over the flattened dense buffer
// (MSDFinalLayer, msd_pytorch/msd_module.py:60-88); its backward materialises a dense
// gradient of the block output, which MSDBlockFunction.backward then clones
// (msd_block.py:83).  Here the layer is two streaming kernels over the same buffers:
//   forward   out[n,o,v]   = b[o] + sum_c W[o,c] result[n,c,v]
//   backward  gradients[n,c,v]  = sum_o W[o,c] gout[n,o,v]     (written straight into the
//                                  buffer the block backward then updates in place: no
//                                  intermediate tensor, no clone)
//             gW[o,c] += sum_{n,v} gout[n,o,v] result[n,c,v],  gb[o] += sum gout[n,o,v]
// Both are HBM-bound: every channel is read (written) once with 128-bit accesses.
// Weight/bias gradients use per-block partials and the fixed-order second pass that the
// fused convolution backward uses (deterministic).
#include "common.cuh"
#include "kernels.h"

namespace msd {
namespace fast {

int sm_count(int device);

constexpr int kMaxFinalOut = 8;   // output channels handled by the tuned kernels
constexpr int kFinalChunk = 8;    // channels per block in the backward kernel
constexpr int kFinalThreads = 256;

struct FinalParams {
    const float *res;
    int64_t r_sn, r_sc, r_sz, r_sy;
    float *out;  // forward: output; backward: gout (read)
    int64_t o_sn, o_sc, o_sz, o_sy;
    float *grad;  // backward: gradients buffer (written)
    int64_t g_sn, g_sc, g_sz, g_sy;
    const float *w;     // [O][C]
    const float *bias;  // [O]
    float *part;        // backward: [vchunks][O][C + 1] partial sums (last column: bias)
    int N, C, O, Z, Y, X;
    int vchunks;
};

__device__ __forceinline__ void unravel_quad(int64_t i, int xq, int Y, int Z, int &n, int &z, int &y, int &x4) {
    x4 = (int)(i % xq);
    int64_t r = i / xq;
    y = (int)(r % Y);
    r /= Y;
    z = (int)(r % Z);
    n = (int)(r / Z);
}

template <int O>
__global__ void __launch_bounds__(kFinalThreads) final_forward_kernel(const FinalParams p) {
    const int xq = p.X / 4;
    const int64_t total = (int64_t)p.N * p.Z * p.Y * xq;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int n, z, y, x4;
        unravel_quad(i, xq, p.Y, p.Z, n, z, y, x4);
        const float *rp = p.res + n * p.r_sn + z * p.r_sz + (int64_t)y * p.r_sy + 4 * x4;
        float4 acc[O];
#pragma unroll
        for (int o = 0; o < O; ++o) {
            const float b = p.bias[o];
            acc[o] = make_float4(b, b, b, b);
        }
#pragma unroll 4
        for (int c = 0; c < p.C; ++c) {
            const float4 v = *reinterpret_cast<const float4 *>(rp + c * p.r_sc);
#pragma unroll
            for (int o = 0; o < O; ++o) {
                const float wv = __ldg(p.w + o * p.C + c);
                acc[o].x = fmaf(wv, v.x, acc[o].x);
                acc[o].y = fmaf(wv, v.y, acc[o].y);
                acc[o].z = fmaf(wv, v.z, acc[o].z);
                acc[o].w = fmaf(wv, v.w, acc[o].w);
            }
        }
        float *op = p.out + n * p.o_sn + z * p.o_sz + (int64_t)y * p.o_sy + 4 * x4;
#pragma unroll
        for (int o = 0; o < O; ++o) *reinterpret_cast<float4 *>(op + o * p.o_sc) = acc[o];
    }
}

// grid = (vchunks, ceil(C / kFinalChunk)).  Block (vc, cc) handles channels
// [cc*8, cc*8+8) on the voxel quads vc, vc + vchunks, ... (strided by block).
template <int O>
__global__ void __launch_bounds__(kFinalThreads) final_backward_kernel(const FinalParams p) {
    const int xq = p.X / 4;
    const int64_t total = (int64_t)p.N * p.Z * p.Y * xq;
    const int c0 = blockIdx.y * kFinalChunk;
    const int nc = min(kFinalChunk, p.C - c0);
    float wl[O][kFinalChunk];
#pragma unroll
    for (int o = 0; o < O; ++o)
#pragma unroll
        for (int k = 0; k < kFinalChunk; ++k) wl[o][k] = k < nc ? p.w[o * p.C + c0 + k] : 0.f;
    float acc[O][kFinalChunk];
    float bacc[O];
#pragma unroll
    for (int o = 0; o < O; ++o) {
        bacc[o] = 0.f;
#pragma unroll
        for (int k = 0; k < kFinalChunk; ++k) acc[o][k] = 0.f;
    }
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int n, z, y, x4;
        unravel_quad(i, xq, p.Y, p.Z, n, z, y, x4);
        const float *gp = p.out + n * p.o_sn + z * p.o_sz + (int64_t)y * p.o_sy + 4 * x4;
        float4 g[O];
#pragma unroll
        for (int o = 0; o < O; ++o) {
            g[o] = *reinterpret_cast<const float4 *>(gp + o * p.o_sc);
            bacc[o] += (g[o].x + g[o].y) + (g[o].z + g[o].w);
        }
        const float *rp = p.res + n * p.r_sn + z * p.r_sz + (int64_t)y * p.r_sy + 4 * x4 + c0 * p.r_sc;
        float *dp = p.grad + n * p.g_sn + z * p.g_sz + (int64_t)y * p.g_sy + 4 * x4 + c0 * p.g_sc;
#pragma unroll
        for (int k = 0; k < kFinalChunk; ++k) {
            if (k < nc) {
                const float4 r = *reinterpret_cast<const float4 *>(rp + k * p.r_sc);
                float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int o = 0; o < O; ++o) {
                    d.x = fmaf(wl[o][k], g[o].x, d.x);
                    d.y = fmaf(wl[o][k], g[o].y, d.y);
                    d.z = fmaf(wl[o][k], g[o].z, d.z);
                    d.w = fmaf(wl[o][k], g[o].w, d.w);
                    acc[o][k] += (g[o].x * r.x + g[o].y * r.y) + (g[o].z * r.z + g[o].w * r.w);
                }
                *reinterpret_cast<float4 *>(dp + k * p.g_sc) = d;
            }
        }
    }
    // block reduction: warp shuffles, then the eight warps in fixed order
    __shared__ float red[kFinalThreads / 32][O * (kFinalChunk + 1)];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 0; o < O; ++o) {
#pragma unroll
        for (int k = 0; k <= kFinalChunk; ++k) {
            float v = k < kFinalChunk ? acc[o][k] : bacc[o];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
            if (lane == 0) red[warp][o * (kFinalChunk + 1) + k] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < O * (kFinalChunk + 1)) {
        const int o = threadIdx.x / (kFinalChunk + 1), k = threadIdx.x % (kFinalChunk + 1);
        float s = 0.f;
#pragma unroll
        for (int wv = 0; wv < kFinalThreads / 32; ++wv) s += red[wv][threadIdx.x];
        float *dst = p.part + ((int64_t)blockIdx.x * p.O + o) * (p.C + 1);
        if (k < kFinalChunk) {
            if (k < nc) dst[c0 + k] = s;
        } else if (blockIdx.y == 0) {
            dst[p.C] = s;  // bias column, once per voxel chunk
        }
    }
}

static bool final_view_ok(const View &v) {
    return v.sx == 1 && (v.sn % 4) == 0 && (v.sc % 4) == 0 && (v.sy % 4) == 0 && (v.sz % 4) == 0 && (((uintptr_t)v.p) & 15) == 0 && (v.x % 4) == 0;
}

bool final_supported(const View &res, const View &out) {
    return out.c >= 1 && out.c <= kMaxFinalOut && res.c >= 1 && final_view_ok(res) && final_view_ok(out) && res.n == out.n && res.z == out.z &&
           res.y == out.y && res.x == out.x;
}

static int final_vchunks(int device, int64_t quads) {
    int64_t v = (int64_t)sm_count(device) * 2;
    const int64_t by_work = ceil_div(quads, kFinalThreads);
    if (v > by_work) v = by_work;
    if (v < 1) v = 1;
    return (int)v;
}

size_t final_workspace_bytes(int64_t c_in, int64_t c_out) { return (size_t)(2 * 256) * c_out * (c_in + 1) * sizeof(float) + 256; }

static void fill(FinalParams &p, const View &res, const View &out) {
    memset(&p, 0, sizeof(p));
    p.res = (const float *)res.p;
    p.r_sn = res.sn, p.r_sc = res.sc, p.r_sz = res.sz, p.r_sy = res.sy;
    p.out = (float *)out.p;
    p.o_sn = out.sn, p.o_sc = out.sc, p.o_sz = out.sz, p.o_sy = out.sy;
    p.N = (int)res.n, p.C = (int)res.c, p.O = (int)out.c, p.Z = (int)res.z, p.Y = (int)res.y, p.X = (int)res.x;
}

template <int O>
static void launch_fwd(const FinalParams &p, int grid, cudaStream_t s) {
    final_forward_kernel<O><<<grid, kFinalThreads, 0, s>>>(p);
}
template <int O>
static void launch_bwd(const FinalParams &p, dim3 grid, cudaStream_t s) {
    final_backward_kernel<O><<<grid, kFinalThreads, 0, s>>>(p);
}

#define DISPATCH_O(fn, ...)                   \
    switch (p.O) {                            \
        case 1: fn<1>(__VA_ARGS__); break;    \
        case 2: fn<2>(__VA_ARGS__); break;    \
        case 3: fn<3>(__VA_ARGS__); break;    \
        case 4: fn<4>(__VA_ARGS__); break;    \
        case 5: fn<5>(__VA_ARGS__); break;    \
        case 6: fn<6>(__VA_ARGS__); break;    \
        case 7: fn<7>(__VA_ARGS__); break;    \
        default: fn<8>(__VA_ARGS__); break;   \
    }

int final_forward(const View &res, const float *w, const float *bias, const View &out, int device, cudaStream_t s) {
    FinalParams p;
    fill(p, res, out);
    p.w = w, p.bias = bias;
    const int64_t quads = res.n * res.z * res.y * (res.x / 4);
    if (quads == 0) return MSD_OK;
    int64_t grid = ceil_div(quads, kFinalThreads);
    const int64_t gmax = (int64_t)sm_count(device) * 8;
    if (grid > gmax) grid = gmax;
    DISPATCH_O(launch_fwd, p, (int)grid, s);
    count_launch(true);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

int final_backward(const View &res, const View &gout, const float *w, const View &grad, float *gw, float *gb, void *ws, size_t wsb, int device,
                   cudaStream_t s) {
    FinalParams p;
    fill(p, res, gout);
    p.w = w;
    p.grad = (float *)grad.p;
    p.g_sn = grad.sn, p.g_sc = grad.sc, p.g_sz = grad.sz, p.g_sy = grad.sy;
    const int64_t quads = res.n * res.z * res.y * (res.x / 4);
    if (quads == 0) return MSD_OK;
    p.vchunks = final_vchunks(device, quads);
    const size_t need = (size_t)p.vchunks * p.O * (p.C + 1) * sizeof(float);
    if (!ws || wsb < need) MSD_FAIL(MSD_ERR_WORKSPACE, "final layer backward: workspace of %zu bytes needed, %zu given", need, wsb);
    p.part = (float *)ws;
    dim3 grid(p.vchunks, (unsigned)ceil_div(p.C, kFinalChunk));
    DISPATCH_O(launch_bwd, p, grid, s);
    count_launch(true);
    MSD_CUDA_TRY(cudaGetLastError());
    // second pass: one entry per output channel; the bias sits behind each row of weight partials
    ReduceList list;
    list.count = 0, list.ws_used = 0;
    for (int o = 0; o < p.O; ++o) {
        // partial row layout is [vchunk][O][C+1]; express output channel o as nk = C values with
        // a pitch of O*(C+1): done by one entry per (o) using a strided view through `pitch`
        ReduceEntry &e = list.e[list.count++];
        e.pk = p.part + (int64_t)o * (p.C + 1);
        e.pb = gb ? p.part + (int64_t)o * (p.C + 1) + p.C : nullptr;
        e.gk = gw ? gw + (int64_t)o * p.C : nullptr;
        e.gb = gb ? gb + o : nullptr;
        e.nparts = p.vchunks;
        e.nk = p.C;
        e.pitch = (int64_t)p.O * (p.C + 1);
        e.pitch_b = e.pitch;
    }
    return flush_reductions(&list, s);
}

}  // namespace fast
}  // namespace msd

// Generic (any dtype / stride / channel count) kernels of the eight MSD convolution ops.
//
// These are the always-correct path: float32 and float64, arbitrary strides,
// any number of input and output channels, any size >= dilation.  The tuned
// sm_100a kernels in fast_forward_2d.cuh / fast_backward.cuh take over for the
// float32, width-1 shapes of the MSD block; everything else lands here.
//
// Arithmetic contract (what the reference's kernels compute):
//   forward     out[n,o,p] = bias[o] + sum_c sum_t in[n,c,refl(p + d t)] k[o,c,t]
//               (conv2d_forward.cu:143-173, conv3d_forward.cu:160-195)
//   backward_x  gin[n,c,q] += sum_o sum_{(p,t): refl(p + d t) = q} gate(p) gout[n,o,p] k[o,c,t]
//               (the exact adjoint; the reference reaches it with a border tap
//               flip, conv2d_backward_x.cu:56-71,153-207)
//   backward_k  gk[o,c,t] += sum_{n,p} in[n,c,refl(p + d t)] gout[n,o,p] gate(p)
//               (conv2d_backward_k.cu:89-111)
//   bias        gb[o]     += sum_{n,p} gout[n,o,p] gate(p)   (conv2d_backward_bias.cu:37-48)
// with gate(p) = out[n,o,p] > 0 for the ReLU variants and 1 otherwise.
// Weight and bias gradients are two-pass and deterministic: pass one writes one
// partial per thread block (warp shuffles, then shared memory), pass two adds
// the partials in a fixed order.
#include "common.cuh"
#include "kernels.h"

namespace msd {
namespace generic {

template <typename T>
struct TV {  // typed view
    T *p;
    int n, c, z, y, x;
    int64_t sn, sc, sz, sy, sx;
};
template <typename T>
static TV<T> typed(const View &v) {
    TV<T> t;
    t.p = (T *)v.p;
    t.n = (int)v.n, t.c = (int)v.c, t.z = (int)v.z, t.y = (int)v.y, t.x = (int)v.x;
    t.sn = v.sn, t.sc = v.sc, t.sz = v.sz, t.sy = v.sy, t.sx = v.sx;
    return t;
}

// Decompose a linear voxel index into (n, z, y, x).
__device__ __forceinline__ void unravel(int64_t i, int Z, int Y, int X, int &n, int &z, int &y, int &x) {
    x = (int)(i % X);
    i /= X;
    y = (int)(i % Y);
    i /= Y;
    z = (int)(i % Z);
    n = (int)(i / Z);
}

template <typename T, int ND, bool RELU>
__global__ void __launch_bounds__(256)
forward_kernel(TV<const T> in, const T *__restrict__ k, const T *__restrict__ bias, TV<T> out, int d, int64_t nvox) {
    constexpr int TZ = (ND == 3) ? 3 : 1;
    constexpr int TAPS = TZ * 9;
    const int C = in.c, O = out.c;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvox; i += (int64_t)gridDim.x * blockDim.x) {
        int n, z, y, x;
        unravel(i, out.z, out.y, out.x, n, z, y, x);
        int64_t oz[3], oy[3], ox[3];
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            oz[t] = (ND == 3) ? reflect(z + (t - 1) * d, in.z) * in.sz : 0;
            oy[t] = reflect(y + (t - 1) * d, in.y) * in.sy;
            ox[t] = reflect(x + (t - 1) * d, in.x) * in.sx;
        }
        const T *inb = in.p + n * in.sn;
        T *outp = out.p + n * out.sn + z * out.sz + y * out.sy + x * out.sx;
        for (int o = 0; o < O; ++o) {
            T acc = bias[o];
            const T *kk = k + (int64_t)o * C * TAPS;
            for (int c = 0; c < C; ++c) {
                const T *ic = inb + c * in.sc;
#pragma unroll
                for (int tz = 0; tz < TZ; ++tz)
#pragma unroll
                    for (int ty = 0; ty < 3; ++ty)
#pragma unroll
                        for (int tx = 0; tx < 3; ++tx)
                            acc += ic[oz[(ND == 3) ? tz : 1] + oy[ty] + ox[tx]] * kk[c * TAPS + (tz * 3 + ty) * 3 + tx];
            }
            if (RELU) acc = acc > T(0) ? acc : T(0);
            outp[o * out.sc] = acc;
        }
    }
}

// For input position q on an axis of size n, the source positions p (and tap
// index t in {0,1,2}) with refl(p + d (t-1)) == q: the direct one p = q - d (t-1)
// if it lies inside, plus one folded source for the taps that can leave the
// image on q's side.  Returns the number of sources (0..2) in src[].
__device__ __forceinline__ int adjoint_sources(int q, int t, int d, int n, int src[2]) {
    int cnt = 0;
    int p = q - d * (t - 1);
    if (p >= 0 && p < n) src[cnt++] = p;
    if (t == 0) {  // p - d = -q - 1  ->  p = d - 1 - q
        p = d - 1 - q;
        if (p >= 0 && p < n) src[cnt++] = p;
    } else if (t == 2) {  // p + d = 2n - 1 - q
        p = 2 * n - 1 - q - d;
        if (p >= 0 && p < n) src[cnt++] = p;
    }
    return cnt;
}

template <typename T, int ND, bool RELU>
__global__ void __launch_bounds__(256)
backward_x_kernel(TV<const T> out, TV<const T> gout, const T *__restrict__ k, TV<T> gin, int d, int64_t nvox) {
    constexpr int TZ = (ND == 3) ? 3 : 1;
    constexpr int TAPS = TZ * 9;
    const int C = gin.c, O = gout.c;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvox; i += (int64_t)gridDim.x * blockDim.x) {
        int n, z, y, x;
        unravel(i, gin.z, gin.y, gin.x, n, z, y, x);
        // Per axis and tap: up to two source positions.
        int sz_[3][2], sy_[3][2], sx_[3][2], nz[3], ny[3], nx[3];
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            if (ND == 3) {
                nz[t] = adjoint_sources(z, t, d, gout.z, sz_[t]);
            } else {
                nz[t] = (t == 1) ? 1 : 0;
                sz_[t][0] = 0;
            }
            ny[t] = adjoint_sources(y, t, d, gout.y, sy_[t]);
            nx[t] = adjoint_sources(x, t, d, gout.x, sx_[t]);
        }
        T *ginp = gin.p + n * gin.sn + z * gin.sz + y * gin.sy + x * gin.sx;
        for (int c = 0; c < C; ++c) {
            T g = 0;
            for (int o = 0; o < O; ++o) {
                const T *go = gout.p + n * gout.sn + o * gout.sc;
                const T *oo = RELU ? out.p + n * out.sn + o * out.sc : nullptr;
                const T *kk = k + ((int64_t)o * C + c) * TAPS;
#pragma unroll
                for (int tz = (ND == 3 ? 0 : 1); tz < (ND == 3 ? 3 : 2); ++tz)
                    for (int a = 0; a < nz[tz]; ++a)
#pragma unroll
                        for (int ty = 0; ty < 3; ++ty)
                            for (int b = 0; b < ny[ty]; ++b)
#pragma unroll
                                for (int tx = 0; tx < 3; ++tx)
                                    for (int e = 0; e < nx[tx]; ++e) {
                                        const int pz = sz_[tz][a], py = sy_[ty][b], px = sx_[tx][e];
                                        T v = go[pz * gout.sz + py * gout.sy + px * gout.sx];
                                        if (RELU) {
                                            if (!(oo[pz * out.sz + py * out.sy + px * out.sx] > T(0))) v = 0;
                                        }
                                        const int kt = ((ND == 3 ? tz : 0) * 3 + ty) * 3 + tx;
                                        g += v * kk[kt];
                                    }
            }
            ginp[c * gin.sc] += g;
        }
    }
}

template <typename T>
__device__ __forceinline__ T warp_sum(T v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
    return v;
}

// Pass one of the weight gradient.  grid = (chunks, O*C); block = 256.
// partial[chunk][(o*C + c)*TAPS + t]
template <typename T, int ND, bool RELU>
__global__ void __launch_bounds__(256)
backward_k_partial_kernel(TV<const T> out, TV<const T> gout, TV<const T> in, T *__restrict__ partial, int d, int64_t nvox) {
    constexpr int TZ = (ND == 3) ? 3 : 1;
    constexpr int TAPS = TZ * 9;
    const int C = in.c;
    const int oc = blockIdx.y;
    const int o = oc / C, c = oc % C;
    T acc[TAPS];
#pragma unroll
    for (int t = 0; t < TAPS; ++t) acc[t] = 0;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvox; i += (int64_t)gridDim.x * blockDim.x) {
        int n, z, y, x;
        unravel(i, gout.z, gout.y, gout.x, n, z, y, x);
        T g = gout.p[n * gout.sn + o * gout.sc + z * gout.sz + y * gout.sy + x * gout.sx];
        if (RELU) {
            if (!(out.p[n * out.sn + o * out.sc + z * out.sz + y * out.sy + x * out.sx] > T(0))) g = 0;
        }
        const T *ic = in.p + n * in.sn + c * in.sc;
        int64_t oz[3], oy[3], ox[3];
#pragma unroll
        for (int t = 0; t < 3; ++t) {
            oz[t] = (ND == 3) ? reflect(z + (t - 1) * d, in.z) * in.sz : 0;
            oy[t] = reflect(y + (t - 1) * d, in.y) * in.sy;
            ox[t] = reflect(x + (t - 1) * d, in.x) * in.sx;
        }
#pragma unroll
        for (int tz = 0; tz < TZ; ++tz)
#pragma unroll
            for (int ty = 0; ty < 3; ++ty)
#pragma unroll
                for (int tx = 0; tx < 3; ++tx)
                    acc[(tz * 3 + ty) * 3 + tx] += ic[oz[(ND == 3) ? tz : 1] + oy[ty] + ox[tx]] * g;
    }
    __shared__ T red[8][TAPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int t = 0; t < TAPS; ++t) {
        T v = warp_sum(acc[t]);
        if (lane == 0) red[warp][t] = v;
    }
    __syncthreads();
    if (threadIdx.x < TAPS) {
        T s = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red[w][threadIdx.x];
        partial[((int64_t)blockIdx.x * gridDim.y + oc) * TAPS + threadIdx.x] = s;
    }
}

// Pass one of the bias gradient.  grid = (chunks, O); partial[chunk][o]
template <typename T, bool RELU>
__global__ void __launch_bounds__(256)
backward_bias_partial_kernel(TV<const T> out, TV<const T> gout, T *__restrict__ partial, int64_t nvox) {
    const int o = blockIdx.y;
    T acc = 0;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvox; i += (int64_t)gridDim.x * blockDim.x) {
        int n, z, y, x;
        unravel(i, gout.z, gout.y, gout.x, n, z, y, x);
        T g = gout.p[n * gout.sn + o * gout.sc + z * gout.sz + y * gout.sy + x * gout.sx];
        if (RELU) {
            if (!(out.p[n * out.sn + o * out.sc + z * out.sz + y * out.sy + x * out.sx] > T(0))) g = 0;
        }
        acc += g;
    }
    __shared__ T red[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T v = warp_sum(acc);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
        T s = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) s += red[w];
        partial[(int64_t)blockIdx.x * gridDim.y + o] = s;
    }
}

// Pass two: dst[j] += sum_{p = 0..nparts-1} partial[p*pitch + j], p ascending.
template <typename T>
__global__ void __launch_bounds__(128)
reduce_partials_kernel(const T *__restrict__ partial, int nparts, int64_t pitch, int64_t nout, T *__restrict__ dst) {
    const int64_t j = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (j >= nout) return;
    T s0 = 0, s1 = 0, s2 = 0, s3 = 0;
    int p = 0;
    for (; p + 3 < nparts; p += 4) {
        s0 += partial[(int64_t)(p + 0) * pitch + j];
        s1 += partial[(int64_t)(p + 1) * pitch + j];
        s2 += partial[(int64_t)(p + 2) * pitch + j];
        s3 += partial[(int64_t)(p + 3) * pitch + j];
    }
    for (; p < nparts; ++p) s0 += partial[(int64_t)p * pitch + j];
    dst[j] += (s0 + s1) + (s2 + s3);
}

static int chunks_for(int64_t nvox, int64_t pairs) {
    // Enough blocks to fill the GPU a few times over, never more than the voxels justify.
    int64_t by_work = ceil_div(nvox, 256 * 4);
    int64_t by_fill = ceil_div(148 * 8, pairs);
    int64_t c = by_work < by_fill ? by_work : by_fill;
    if (c < 1) c = 1;
    if (c > 1024) c = 1024;
    return (int)c;
}

size_t workspace_bytes(int dtype, int nd, int64_t nvox, int64_t c_in, int64_t c_out) {
    const size_t es = dtype == MSD_F64 ? 8 : 4;
    const int taps = nd == 3 ? 27 : 9;
    const size_t k = (size_t)chunks_for(nvox, c_in * c_out) * c_in * c_out * taps * es;
    const size_t b = (size_t)chunks_for(nvox, c_out) * c_out * es;
    return (k > b ? k : b) + 256;
}

static int grid_for(int64_t nvox) {
    int64_t g = ceil_div(nvox, 256);
    if (g > (1 << 30)) g = 1 << 30;
    return (int)g;
}

template <typename T>
static int forward_t(bool relu, const View &in, const void *k, const void *bias, const View &out, int nd, int d, cudaStream_t s) {
    const int64_t nvox = out.n * out.z * out.y * out.x;
    if (nvox == 0 || out.c == 0) return MSD_OK;
    auto i = typed<const T>(in);
    auto o = typed<T>(out);
    const int g = grid_for(nvox);
#define L(ND, R) forward_kernel<T, ND, R><<<g, 256, 0, s>>>(i, (const T *)k, (const T *)bias, o, d, nvox)
    if (nd == 2) {
        if (relu) L(2, true); else L(2, false);
    } else {
        if (relu) L(3, true); else L(3, false);
    }
#undef L
    count_launch(false);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

int forward(int dtype, bool relu, const View &in, const void *k, const void *bias, const View &out, int nd, int d, cudaStream_t s) {
    return dtype == MSD_F64 ? forward_t<double>(relu, in, k, bias, out, nd, d, s) : forward_t<float>(relu, in, k, bias, out, nd, d, s);
}

template <typename T>
static int backward_x_t(bool relu, const View *out, const View &gout, const void *k, const View &gin, int nd, int d, cudaStream_t s) {
    const int64_t nvox = gin.n * gin.z * gin.y * gin.x;
    if (nvox == 0 || gin.c == 0) return MSD_OK;
    auto go = typed<const T>(gout);
    auto oo = relu ? typed<const T>(*out) : go;
    auto gi = typed<T>(gin);
    const int g = grid_for(nvox);
#define L(ND, R) backward_x_kernel<T, ND, R><<<g, 256, 0, s>>>(oo, go, (const T *)k, gi, d, nvox)
    if (nd == 2) {
        if (relu) L(2, true); else L(2, false);
    } else {
        if (relu) L(3, true); else L(3, false);
    }
#undef L
    count_launch(false);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

int backward_x(int dtype, bool relu, const View *out, const View &gout, const void *k, const View &gin, int nd, int d, cudaStream_t s) {
    return dtype == MSD_F64 ? backward_x_t<double>(relu, out, gout, k, gin, nd, d, s) : backward_x_t<float>(relu, out, gout, k, gin, nd, d, s);
}

template <typename T>
static int backward_k_t(bool relu, const View *out, const View &gout, const View &in, void *gk, int nd, int d, void *ws, size_t wsb, cudaStream_t s) {
    const int64_t nvox = gout.n * gout.z * gout.y * gout.x;
    const int64_t pairs = gout.c * in.c;
    if (pairs == 0) return MSD_OK;
    const int taps = nd == 3 ? 27 : 9;
    const int chunks = chunks_for(nvox, pairs);
    const size_t need = (size_t)chunks * pairs * taps * sizeof(T);
    if (!ws || wsb < need) MSD_FAIL(MSD_ERR_WORKSPACE, "backward_k: workspace of %zu bytes needed, %zu given", need, wsb);
    if (pairs > 65535) MSD_FAIL(MSD_ERR_UNSUPPORTED, "backward_k: c_in*c_out = %lld exceeds 65535", (long long)pairs);
    auto go = typed<const T>(gout);
    auto oo = relu ? typed<const T>(*out) : go;
    auto ii = typed<const T>(in);
    dim3 grid(chunks, (unsigned)pairs);
#define L(ND, R) backward_k_partial_kernel<T, ND, R><<<grid, 256, 0, s>>>(oo, go, ii, (T *)ws, d, nvox)
    if (nd == 2) {
        if (relu) L(2, true); else L(2, false);
    } else {
        if (relu) L(3, true); else L(3, false);
    }
#undef L
    count_launch(false);
    MSD_CUDA_TRY(cudaGetLastError());
    const int64_t nout = pairs * taps;
    reduce_partials_kernel<T><<<(unsigned)ceil_div(nout, 128), 128, 0, s>>>((const T *)ws, chunks, nout, nout, (T *)gk);
    count_launch(false);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

int backward_k(int dtype, bool relu, const View *out, const View &gout, const View &in, void *gk, int nd, int d, void *ws, size_t wsb, cudaStream_t s) {
    return dtype == MSD_F64 ? backward_k_t<double>(relu, out, gout, in, gk, nd, d, ws, wsb, s)
                            : backward_k_t<float>(relu, out, gout, in, gk, nd, d, ws, wsb, s);
}

template <typename T>
static int backward_bias_t(bool relu, const View *out, const View &gout, void *gb, void *ws, size_t wsb, cudaStream_t s) {
    const int64_t nvox = gout.n * gout.z * gout.y * gout.x;
    const int64_t O = gout.c;
    if (O == 0) return MSD_OK;
    const int chunks = chunks_for(nvox, O);
    const size_t need = (size_t)chunks * O * sizeof(T);
    if (!ws || wsb < need) MSD_FAIL(MSD_ERR_WORKSPACE, "backward_bias: workspace of %zu bytes needed, %zu given", need, wsb);
    if (O > 65535) MSD_FAIL(MSD_ERR_UNSUPPORTED, "backward_bias: c_out = %lld exceeds 65535", (long long)O);
    auto go = typed<const T>(gout);
    auto oo = relu ? typed<const T>(*out) : go;
    dim3 grid(chunks, (unsigned)O);
    if (relu)
        backward_bias_partial_kernel<T, true><<<grid, 256, 0, s>>>(oo, go, (T *)ws, nvox);
    else
        backward_bias_partial_kernel<T, false><<<grid, 256, 0, s>>>(oo, go, (T *)ws, nvox);
    count_launch(false);
    MSD_CUDA_TRY(cudaGetLastError());
    reduce_partials_kernel<T><<<(unsigned)ceil_div(O, 128), 128, 0, s>>>((const T *)ws, chunks, O, O, (T *)gb);
    count_launch(false);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

int reduce_partials_f32(const float *partial, int nparts, int64_t pitch, int64_t nout, float *dst, cudaStream_t s) {
    reduce_partials_kernel<float><<<(unsigned)ceil_div(nout, 128), 128, 0, s>>>(partial, nparts, pitch, nout, dst);
    count_launch(false);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

int backward_bias(int dtype, bool relu, const View *out, const View &gout, void *gb, void *ws, size_t wsb, cudaStream_t s) {
    return dtype == MSD_F64 ? backward_bias_t<double>(relu, out, gout, gb, ws, wsb, s) : backward_bias_t<float>(relu, out, gout, gb, ws, wsb, s);
}

}  // namespace generic
}  // namespace msd

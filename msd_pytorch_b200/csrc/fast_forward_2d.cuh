// Forward of one 2D MSD layer that emits ONE channel (float32):
//     out[y][x] = [relu]( bias + sum_c sum_{ty,tx} k[c][ty][tx] * in[c][refl(y + (ty-1) D)][refl(x + (tx-1) D)] )
// (what conv2d_forward.cu:95-174 of the reference computes, for c_out = 1).
//
// Data movement (sm_100a): a producer warp issues ONE tiled TMA load
// (cp.async.bulk.tensor.4d, completion on an mbarrier) per input channel: the output tile
// plus a halo of D rows and D (rounded up to 4, for the 16-byte rule) columns.  Out-of-image
// parts of the box are zero-filled by the TMA unit.  The boxes land in a multi-stage
// shared-memory ring; the producer runs up to `stages` channels ahead, across tile
// boundaries.  Blocks are persistent and take tiles in a fixed round-robin order.
//
// Compute: the tile has Q*R*D rows and 128 columns.  A warp owns the rows
// {base + i + j*D, j < R} of one residue class i modulo D ("row lattice") and its 32 lanes
// own K column segments 32 apart.  Output rows j and j+1 of a lattice share two of their
// three input rows, so per channel a thread loads (R+2)*3*K values from shared memory for
// R*9*K FMAs.  All shared loads are scalar with lanes on consecutive columns (conflict
// free for any D).
//
// Reflection: rows are handled for free by giving every thread the (possibly reflected)
// shared-memory row of each of its R+2 lattice rows in a register.  Columns: in tiles that
// touch the left or right image border the x-D tap of the first segment and the x+D taps
// use per-thread offsets that point at the mirror cell (always inside the same box); all
// other tiles run a copy of the loop with compile-time offsets.
#pragma once
#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace msd {
namespace fast {

constexpr int kFwdTW = 128;  // tile width
constexpr int kFwdMaxStages = 8;

struct Fwd2dParams {
    float *out;
    int64_t out_sn, out_sy;
    const float *k;     // [C][9]
    const float *bias;  // [1]
    int N, C, Y, X;
    int tiles_x, tiles_y;
    long long num_tiles;
    int stages;
    int relu;
    int *status;
};

template <int D, int R, int Q, int K>
struct Fwd2dCfg {
    static constexpr int XW = kFwdTW / (32 * K);    // warps side by side along x
    static constexpr int NCW = Q * D * XW;          // compute warps
    static constexpr int THREADS = NCW * 32 + 32;   // + producer warp
    static constexpr int TH = Q * R * D;            // tile rows
    static constexpr int DP = (D + 3) & ~3;
    static constexpr int BW = kFwdTW + 2 * DP;      // box columns
    static constexpr int BH = TH + 2 * D;           // box rows
    static constexpr int STAGE_BYTES = ((BH * BW * 4) + 127) & ~127;
    static constexpr int STAGE = STAGE_BYTES / 4;
};

// One input channel's contribution to a thread's R x K accumulators.  `rp[m]` points at the
// thread's first column in lattice row m of the box; BORDER selects run-time column
// offsets for the taps that may leave the image.
template <int D, int R, int K, bool BORDER>
__device__ __forceinline__ void fwd2d_channel(float (&acc)[R][K], const float *st, const int (&rowoff)[R + 2], const float *wsm_c, int dl,
                                              const int (&dr)[K]) {
    const float4 *wp = reinterpret_cast<const float4 *>(wsm_c);
    const float4 w0 = wp[0], w1 = wp[1], w2 = wp[2];
    const float w[9] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w, w2.x};
#pragma unroll
    for (int m = 0; m < R + 2; ++m) {
        const float *rp = st + rowoff[m];
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const float a = (BORDER && k == 0) ? rp[dl] : rp[32 * k - D];
            const float b = rp[32 * k];
            const float cc = BORDER ? rp[32 * k + dr[k]] : rp[32 * k + D];
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const int t = m - j;  // tap row of output row j that reads lattice row m
                if (t >= 0 && t <= 2) {
                    acc[j][k] = fmaf(w[t * 3 + 0], a, acc[j][k]);
                    acc[j][k] = fmaf(w[t * 3 + 1], b, acc[j][k]);
                    acc[j][k] = fmaf(w[t * 3 + 2], cc, acc[j][k]);
                }
            }
        }
    }
}

template <int D, int R, int Q, int K>
__global__ void __launch_bounds__(Fwd2dCfg<D, R, Q, K>::THREADS, 1)
forward2d_kernel(const __grid_constant__ CUtensorMap map, const Fwd2dParams p) {
    using Cfg = Fwd2dCfg<D, R, Q, K>;
    constexpr int NCW = Cfg::NCW, XW = Cfg::XW, TH = Cfg::TH, DP = Cfg::DP, BW = Cfg::BW, BH = Cfg::BH, STAGE = Cfg::STAGE;
    constexpr int TW = kFwdTW;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t *empty = full + kFwdMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kFwdMaxStages);
    const int wfloats = (p.C * 12 + 31) & ~31;
    float *ring = reinterpret_cast<float *>(smem_raw + 256);
    float *wsm = ring + (size_t)p.stages * STAGE;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            tma::mbar_init(&full[s], 1);
            tma::mbar_init(&empty[s], NCW);
        }
        *abort_flag = 0;
        tma::fence_barrier_init();
        tma::prefetch_tensormap(&map);
    }
    for (int i = tid; i < wfloats; i += Cfg::THREADS) {
        const int c = i / 12, t = i % 12;
        wsm[i] = (c < p.C && t < 9) ? p.k[c * 9 + t] : 0.f;
    }
    __syncthreads();

    const long long tiles_per_image = (long long)p.tiles_x * p.tiles_y;

    if (warp == NCW) {
        // ------------------------------ producer warp ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const int n = (int)(tile / tiles_per_image);
                const int bx = tx_i * TW - DP, by = ty_i * TH - D;
                for (int c = 0; c < p.C; ++c, ++it) {
                    const int s = it % S;
                    if (it >= (uint32_t)S) tma::wait_parity(&empty[s], ((it / S) & 1u) ^ 1u, abort_flag, p.status, 3);
                    tma::mbar_arrive_expect_tx(&full[s], BH * BW * 4);
                    tma::tensor_g2s_4d(ring + (size_t)s * STAGE, &map, bx, by, c, n, &full[s]);
                }
            }
        }
        return;  // every box this warp requested is awaited by the compute warps
    }

    // -------------------------------- compute warps --------------------------------
    const int xw = warp % XW, u = warp / XW;
    const int q = u / D, i = u - q * D;
    const int cb = xw * 32 * K + lane;  // first column of this thread inside the tile
    const float bias = p.bias[0];
    uint32_t it = 0;
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        const int tx_i = (int)(tile % p.tiles_x);
        const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
        const int n = (int)(tile / tiles_per_image);
        const int x0 = tx_i * TW, y0 = ty_i * TH;

        // Shared-memory offset of each lattice row (reflected at the top/bottom border and
        // clamped for rows that only feed outputs below the image).
        int rowoff[R + 2];
#pragma unroll
        for (int m = 0; m < R + 2; ++m) {
            int y = y0 - D + q * R * D + i + m * D;  // image row of lattice row m
            if (y < 0) y = -y - 1;
            if (y >= p.Y) y = 2 * p.Y - 1 - y;
            int br = y - (y0 - D);
            br = br < 0 ? 0 : (br > BH - 1 ? BH - 1 : br);
            rowoff[m] = br * BW + DP + cb;
        }
        // Column offsets of the taps that may leave the image (see fwd2d_channel).
        const bool border = (x0 == 0) || (x0 + TW + D > p.X);
        int dl = -D, dr[K];
        if (x0 == 0 && cb < D) dl = D - 1 - 2 * cb;  // x - D < 0 mirrors to D - 1 - x
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int x = x0 + cb + 32 * k;
            dr[k] = (x < p.X && x + D >= p.X) ? 2 * p.X - 1 - 2 * x - D : D;  // x + D >= X mirrors to 2X - 1 - (x + D)
        }

        float acc[R][K];
#pragma unroll
        for (int j = 0; j < R; ++j)
#pragma unroll
            for (int k = 0; k < K; ++k) acc[j][k] = bias;

        for (int c = 0; c < p.C; ++c, ++it) {
            const int s = it % S;
            tma::wait_parity(&full[s], (it / S) & 1u, abort_flag, p.status, 4);
            const float *st = ring + (size_t)s * STAGE;
            if (border)
                fwd2d_channel<D, R, K, true>(acc, st, rowoff, wsm + c * 12, dl, dr);
            else
                fwd2d_channel<D, R, K, false>(acc, st, rowoff, wsm + c * 12, dl, dr);
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&empty[s]);
        }

        if (!*abort_flag) {
            float *ob = p.out + n * p.out_sn;
#pragma unroll
            for (int j = 0; j < R; ++j) {
                const int y = y0 + q * R * D + i + j * D;
                if (y < p.Y) {
#pragma unroll
                    for (int k = 0; k < K; ++k) {
                        const int x = x0 + cb + 32 * k;
                        float v = acc[j][k];
                        if (p.relu) v = v > 0.f ? v : 0.f;
                        if (x < p.X) ob[(int64_t)y * p.out_sy + x] = v;
                    }
                }
            }
        }
    }
}

typedef int (*Fwd2dLaunchFn)(const CUtensorMap &, const Fwd2dParams &, int grid, int stages, cudaStream_t);
struct Fwd2dVariant {
    Fwd2dLaunchFn launch;
    int threads, th, bh, bw, stage_bytes;
};

}  // namespace fast
}  // namespace msd

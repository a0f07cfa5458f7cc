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
// Compute: the tile has Q*R*D rows and TW (128 or 64) columns.  A warp owns the rows
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
//
// 3D layers (NT = 3) run the same kernel once per z-plane: from one staged 2D tile of
// in[c][z'] a thread accumulates the three in-plane 3x3 sums u_tz[z'] (one per z-tap, 27
// FMAs per loaded lattice value triple), written to a scratch buffer; a second, purely
// streaming kernel then forms out[z] = [relu](bias + u_0[refl(z-D)] + u_1[z] + u_2[refl(z+D)])
// (conv3d_forward.cu:110-196 of the reference, sum re-associated by z-tap).  This keeps the
// staged tiles two-dimensional (a three-dimensional halo for D = 10 does not fit in shared
// memory) and raises the FMA : shared-load ratio to 6.
#pragma once
#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace msd {
namespace fast {

constexpr int kFwdMaxStages = 8;

// Floats of shared memory per input channel for the weights: 9 (27) padded to whole 16-byte
// vectors.  (Storing every weight twice, so that a 128-bit load yields ready-made operand
// pairs of the packed FMA, was measured: 12 % slower in 3D, no gain in 2D.)
__host__ __device__ constexpr int fwd_weight_floats(int nt) { return nt == 3 ? 28 : 12; }

struct Fwd2dParams {
    float *out;          // NT == 1: the output channel; NT == 3: scratch u[3][N][Z][Y][X]
    int64_t out_st, out_sn, out_sz, out_sy;
    const float *k;     // [C][NT*9]
    const float *bias;  // [1]
    int N, C, Z, Y, X;
    int z0, ZW;  // planes [z0, z0 + ZW) are computed (the whole volume unless a z-slab window is set)
    int tiles_x, tiles_y;
    long long num_tiles;
    int stages;
    int relu;
    int *status;
};

template <int D, int R, int Q, int K, int TW>
struct Fwd2dCfg {
    static constexpr int XW = TW / (32 * K);        // warps side by side along x
    static constexpr int NCW = Q * D * XW;          // compute warps
    static constexpr int THREADS = NCW * 32 + 32;   // + producer warp
    static constexpr int TH = Q * R * D;            // tile rows
    static constexpr int DP = (D + 3) & ~3;
    static constexpr int BW = TW + 2 * DP;          // box columns
    static constexpr int BH = TH + 2 * D;           // box rows
    static constexpr int STAGE_BYTES = ((BH * BW * 4) + 127) & ~127;
    static constexpr int STAGE = STAGE_BYTES / 4;
};

// One input channel's contribution to a thread's NT x R x K accumulators.  `rowoff[m]` is the
// offset of the thread's first column in lattice row m of the box; BORDER selects run-time
// column offsets for the taps that may leave the image.
//
// The FMAs are issued as packed pairs (fma.rn.f32x2 through __ffma2_rn): the accumulators of
// two column segments share one instruction, the weight is duplicated into both halves once
// per channel.  Each half is an ordinary fp32 FMA, so results are unchanged; what changes
// is that the 9 (27) multiply-adds per loaded triple take half the issue slots, which is
// what bounds these kernels after the shared-memory loads.
template <int D, int R, int K, int NT, bool BORDER>
__device__ __forceinline__ void fwd2d_channel(float2 (&acc)[NT][R][K / 2], const float *st, const int (&rowoff)[R + 2], const float *wsm_c, int dl,
                                              const int (&dr)[K]) {
    static_assert(K % 2 == 0, "column segments are processed in pairs");
    constexpr int WP = fwd_weight_floats(NT);
    float2 w[NT * 9];
    const float4 *wp = reinterpret_cast<const float4 *>(wsm_c);
#pragma unroll
    for (int i = 0; i < WP / 4; ++i) {
        const float4 t4 = wp[i];
        if (4 * i + 0 < NT * 9) w[4 * i + 0] = make_float2(t4.x, t4.x);
        if (4 * i + 1 < NT * 9) w[4 * i + 1] = make_float2(t4.y, t4.y);
        if (4 * i + 2 < NT * 9) w[4 * i + 2] = make_float2(t4.z, t4.z);
        if (4 * i + 3 < NT * 9) w[4 * i + 3] = make_float2(t4.w, t4.w);
    }
#pragma unroll
    for (int m = 0; m < R + 2; ++m) {
        const float *rp = st + rowoff[m];
#pragma unroll
        for (int kp = 0; kp < K / 2; ++kp) {
            const int k0 = 2 * kp, k1 = 2 * kp + 1;
            float2 a, b, cc;
            a.x = (BORDER && k0 == 0) ? rp[dl] : rp[32 * k0 - D];
            a.y = rp[32 * k1 - D];
            b.x = rp[32 * k0];
            b.y = rp[32 * k1];
            cc.x = BORDER ? rp[32 * k0 + dr[k0]] : rp[32 * k0 + D];
            cc.y = BORDER ? rp[32 * k1 + dr[k1]] : rp[32 * k1 + D];
            // One loaded pair feeds up to 3 * NT accumulators: issuing those FMAs back to back
            // lets consecutive instructions share a source operand (fewer register-file reads;
            // three distinct register pairs per packed FMA run at ~2/3 of the pipe's rate).
            // Every accumulator still receives its terms in the order a, b, c.
#pragma unroll
            for (int tx = 0; tx < 3; ++tx) {
                const float2 v = tx == 0 ? a : (tx == 1 ? b : cc);
#pragma unroll
                for (int j = 0; j < R; ++j) {
                    const int t = m - j;  // tap row of output row j that reads lattice row m
                    if (t >= 0 && t <= 2) {
#pragma unroll
                        for (int tz = 0; tz < NT; ++tz) acc[tz][j][kp] = __ffma2_rn(w[tz * 9 + t * 3 + tx], v, acc[tz][j][kp]);
                    }
                }
            }
        }
    }
}

template <int D, int R, int Q, int K, int NT, int TW>
__global__ void __launch_bounds__(Fwd2dCfg<D, R, Q, K, TW>::THREADS, 1)
forward2d_kernel(const __grid_constant__ CUtensorMap map, const Fwd2dParams p) {
    constexpr int WP = fwd_weight_floats(NT);
    using Cfg = Fwd2dCfg<D, R, Q, K, TW>;
    constexpr int NCW = Cfg::NCW, XW = Cfg::XW, TH = Cfg::TH, DP = Cfg::DP, BW = Cfg::BW, BH = Cfg::BH, STAGE = Cfg::STAGE;

    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t *empty = full + kFwdMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kFwdMaxStages);
    const int wfloats = (p.C * WP + 31) & ~31;
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
        const int c = i / WP, t = i % WP;
        wsm[i] = (c < p.C && t < NT * 9) ? p.k[c * NT * 9 + t] : 0.f;
    }
    tma::allow_dependents();
    __syncthreads();
    // everything above only touched this layer's constants; the channels below were written by
    // the previous layer's kernel
    tma::grid_dependency_wait();

    const long long tiles_per_image = (long long)p.tiles_x * p.tiles_y;

    if (warp == NCW) {
        // ------------------------------ producer warp ------------------------------
        if (lane == 0) {
            uint32_t it = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const long long nz = tile / tiles_per_image;
                const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
                const int bx = tx_i * TW - DP, by = ty_i * TH - D;
                for (int c = 0; c < p.C; ++c, ++it) {
                    const int s = it % S;
                    if (it >= (uint32_t)S) tma::wait_parity(&empty[s], ((it / S) & 1u) ^ 1u, abort_flag, p.status, 3);
                    tma::mbar_arrive_expect_tx(&full[s], BH * BW * 4);
                    if (NT == 3)
                        tma::tensor_g2s_5d(ring + (size_t)s * STAGE, &map, bx, by, z, c, n, &full[s]);
                    else
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
        const long long nz = tile / tiles_per_image;
        const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
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

        float2 acc[NT][R][K / 2];
#pragma unroll
        for (int tz = 0; tz < NT; ++tz)
#pragma unroll
            for (int j = 0; j < R; ++j)
#pragma unroll
                for (int kp = 0; kp < K / 2; ++kp) acc[tz][j][kp] = (NT == 1) ? make_float2(bias, bias) : make_float2(0.f, 0.f);

        for (int c = 0; c < p.C; ++c, ++it) {
            const int s = it % S;
            tma::wait_parity(&full[s], (it / S) & 1u, abort_flag, p.status, 4);
            const float *st = ring + (size_t)s * STAGE;
            if (border)
                fwd2d_channel<D, R, K, NT, true>(acc, st, rowoff, wsm + c * WP, dl, dr);
            else
                fwd2d_channel<D, R, K, NT, false>(acc, st, rowoff, wsm + c * WP, dl, dr);
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&empty[s]);
        }

        if (!*abort_flag) {
#pragma unroll
            for (int tz = 0; tz < NT; ++tz) {
                float *ob = p.out + tz * p.out_st + n * p.out_sn + z * p.out_sz;
#pragma unroll
                for (int j = 0; j < R; ++j) {
                    const int y = y0 + q * R * D + i + j * D;
                    if (y < p.Y) {
#pragma unroll
                        for (int k = 0; k < K; ++k) {
                            const int x = x0 + cb + 32 * k;
                            float v = (k & 1) ? acc[tz][j][k / 2].y : acc[tz][j][k / 2].x;
                            if (NT == 1 && p.relu) v = v > 0.f ? v : 0.f;
                            if (x < p.X) ob[(int64_t)y * p.out_sy + x] = v;
                        }
                    }
                }
            }
        }
    }
}

// Second kernel of the 3D forward: out[n][z][y][x] = [relu](bias + u0[refl(z-d)] + u1[z] + u2[refl(z+d)]),
// u dense [3][N][Z][Y][X], four voxels per thread.
__global__ void __launch_bounds__(256)
zgather_kernel(const float *__restrict__ u, float *__restrict__ out, int64_t out_sn, int64_t out_sz, int64_t out_sy, const float *__restrict__ bias,
               int N, int Z, int Y, int X, int z0, int ZW, int d, int relu) {
    const int xq = X / 4;
    const int64_t total = (int64_t)N * ZW * Y * xq;
    const int64_t plane = (int64_t)Y * X, vol = plane * Z, ust = vol * N;
    const float b = bias[0];
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int x4 = (int)(i % xq);
        int64_t r = i / xq;
        const int y = (int)(r % Y);
        r /= Y;
        const int z = z0 + (int)(r % ZW), n = (int)(r / ZW);
        const int zm = reflect(z - d, Z), zp = reflect(z + d, Z);
        const int64_t off = (int64_t)n * vol + (int64_t)y * X + 4 * x4;
        const float4 a0 = *reinterpret_cast<const float4 *>(u + off + zm * plane);
        const float4 a1 = *reinterpret_cast<const float4 *>(u + ust + off + z * plane);
        const float4 a2 = *reinterpret_cast<const float4 *>(u + 2 * ust + off + zp * plane);
        float4 v;
        v.x = b + a0.x + a1.x + a2.x;
        v.y = b + a0.y + a1.y + a2.y;
        v.z = b + a0.z + a1.z + a2.z;
        v.w = b + a0.w + a1.w + a2.w;
        if (relu) {
            v.x = v.x > 0.f ? v.x : 0.f;
            v.y = v.y > 0.f ? v.y : 0.f;
            v.z = v.z > 0.f ? v.z : 0.f;
            v.w = v.w > 0.f ? v.w : 0.f;
        }
        *reinterpret_cast<float4 *>(out + n * out_sn + z * out_sz + (int64_t)y * out_sy + 4 * x4) = v;
    }
}

typedef int (*Fwd2dLaunchFn)(const CUtensorMap &, const Fwd2dParams &, int grid, int stages, cudaStream_t);
struct Fwd2dVariant {
    Fwd2dLaunchFn launch;
    int threads, th, tw, bh, bw, stage_bytes;
};

}  // namespace fast
}  // namespace msd

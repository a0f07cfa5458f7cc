// Fused backward of one MSD layer that emits ONE channel (float32), 2D and 3D.
//
// For the layer's single output channel let m = gout * [out > 0] (or gout when there is
// no gate).  For every input channel c the layer needs
//     gin[c][q]  += sum_t k[c][t] * M_t[q]                       (input gradient)
//     gk[c][t]   += sum_q in[c][q] * M_t[q]                      (weight gradient)
//     gb         += sum_q m[q]                                   (bias gradient)
// with  M_t[q] = sum of m over the source positions p whose tap t reads q in the forward
// pass, refl(p + d (t - 1)) == q.  Away from the border that is the single position
// q - d (t - 1); near it the edge-inclusive reflection folds a second source in.  (The
// reference reaches the same adjoint with its border tap flip, conv2d_backward_x.cu:56-71,
// and computes the weight gradient in the forward direction, conv2d_backward_k.cu:89-111;
// both sums are re-associated here.)
//
// M_t[q] depends on the layer, not on c.  Each thread therefore computes the 9 (27) values
// M_t of its own voxels ONCE per tile, keeps them in registers, and then streams all C
// input channels past them: per channel one 128-bit load of in[c] and of gin[c], 2 x 9
// (2 x 27) FMAs per voxel, one 128-bit store.  No halo is needed for the C-channel
// streams; only the single channel m is read with a halo, once per tile.
//
// Data movement (sm_100a): a producer warp issues tiled TMA loads
// (cp.async.bulk.tensor, completion on mbarriers) of the tile of in[c] and of gin[c] into a
// multi-stage shared-memory ring, running up to `stages` channels ahead, across tile
// boundaries; eight consumer warps read the ring with 128-bit shared loads and write
// gin[c] straight from registers with 128-bit global stores.  Blocks are persistent and
// take tiles in a fixed round-robin order.
//
// Weight gradient reduction (deterministic, two passes): per channel each warp sums its
// threads' 9 (27) partials with a shuffle reduce-scatter and adds them to its own slot in
// shared memory; at the end of the block the eight warp slots are added in warp order and
// written to `part_k[block]`; a second kernel adds the blocks' partials in block order.
#pragma once
#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace msd {
namespace fast {

constexpr int kConsumerWarps = 8;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kBwdThreads = kConsumers + 32;  // + one producer warp
constexpr int kMaxStages = 8;

struct BwdParams {
    const float *out;  // gate channel or null
    int64_t out_sn, out_sz, out_sy;
    const float *gout;
    int64_t go_sn, go_sz, go_sy;
    const float *in;
    int64_t in_sn, in_sc, in_sz, in_sy;
    float *gin;
    int64_t gi_sn, gi_sc, gi_sz, gi_sy;
    const float *k;  // [C][TAPS]
    float *part_k;   // [grid][C*TAPS]
    float *part_b;   // [grid] or null
    int N, C, Z, Y, X;
    int d, Dp;  // dilation and dilation rounded up to a multiple of 4
    int tiles_x, tiles_y;
    long long num_tiles;
    int stages;
    int *status;
};

template <int ND>
struct BwdTraits {
    static constexpr int RT = (ND == 3) ? 9 : 3;     // row taps: (tz,ty) or ty
    static constexpr int TAPS = RT * 3;
    static constexpr int TAPS_PAD = (ND == 3) ? 28 : 12;  // padded to whole float4s
    static constexpr int NV = (ND == 3) ? 32 : 16;        // reduce-scatter width
};

// Source positions p on an axis of size n with refl(p + d (t-1)) == q; t in {0,1,2}.
__device__ __forceinline__ int adjoint_sources_dev(int q, int t, int d, int n, int src[2]) {
    int cnt = 0;
    int p = q - d * (t - 1);
    if (p >= 0 && p < n) src[cnt++] = p;
    if (t == 0) {
        p = d - 1 - q;
        if (p >= 0 && p < n) src[cnt++] = p;
    } else if (t == 2) {
        p = 2 * n - 1 - q - d;
        if (p >= 0 && p < n) src[cnt++] = p;
    }
    return cnt;
}

// After the call, lane l of the warp holds in the return value the sum over all 32 lanes
// of v[l] (NV == 32) or of v[l & 15] (NV == 16).
template <int NV>
__device__ __forceinline__ float warp_reduce_scatter(float (&v)[NV], int lane) {
#pragma unroll
    for (int h = NV / 2; h >= 1; h >>= 1) {
        const bool up = (lane & h) != 0;
#pragma unroll
        for (int i = 0; i < h; ++i) {
            const float send = up ? v[i] : v[i + h];
            const float keep = up ? v[i + h] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, h);
        }
    }
    float r = v[0];
    if (NV == 16) r += __shfl_xor_sync(0xffffffffu, r, 16);
    return r;
}

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

template <int ND, int TXQ, int J, bool DO_X, bool DO_K>
__global__ void __launch_bounds__(kBwdThreads, 1)
fused_backward_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_gin, const BwdParams p) {
    using T = BwdTraits<ND>;
    constexpr int RT = T::RT, TAPS = T::TAPS, TAPS_PAD = T::TAPS_PAD, NV = T::NV;
    constexpr int TX = TXQ * 4;
    constexpr int RPP = kConsumers / TXQ;  // rows per pass
    constexpr int TR = RPP * J;            // rows per tile
    constexpr int P = 4 * J;               // voxels per thread
    constexpr int NARR = (DO_X ? 1 : 0) + (DO_K ? 1 : 0);
    constexpr int STAGE = NARR * TR * TX;  // floats per ring stage

    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t *empty = full + kMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(empty + kMaxStages);
    float *red = reinterpret_cast<float *>(smem_raw + 192);  // 16 floats
    float *wsm = reinterpret_cast<float *>(smem_raw + 256);
    const int TXP = TX + 2 * p.Dp;
    float *wacc = wsm + (DO_X ? p.C * TAPS_PAD : 0);
    float *rows = wacc + (DO_K ? kConsumerWarps * p.C * TAPS_PAD : 0);
    // ring stages are TMA destinations: 128-byte aligned
    float *ring = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(rows + RT * TR * TXP) + 127) & ~uintptr_t(127));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            tma::mbar_init(&full[s], 1);
            tma::mbar_init(&empty[s], kConsumerWarps);
        }
        *abort_flag = 0;
        tma::fence_barrier_init();
    }
    if (DO_X) {
        for (int i = tid; i < p.C * TAPS_PAD; i += kBwdThreads) {
            const int c = i / TAPS_PAD, t = i % TAPS_PAD;
            wsm[i] = t < TAPS ? p.k[c * TAPS + t] : 0.f;
        }
    }
    if (DO_K) {
        for (int i = tid; i < kConsumerWarps * p.C * TAPS_PAD; i += kBwdThreads) wacc[i] = 0.f;
    }
    __syncthreads();

    const long long tiles_per_plane = (long long)p.tiles_x * p.tiles_y;

    if (warp == kConsumerWarps) {
        // ------------------------------ producer warp ------------------------------
        // One tiled TMA load per array and channel: the TR x TX tile of in[c] and of gin[c].
        // Parts of the box beyond the image are zero-filled by the TMA unit.
        if (lane == 0) {
            if (DO_K) tma::prefetch_tensormap(&map_in);
            if (DO_X) tma::prefetch_tensormap(&map_gin);
            uint32_t it = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const long long nz = tile / tiles_per_plane;
                const int z = (int)(nz % p.Z), n = (int)(nz / p.Z);
                const int x0 = tx_i * TX, y0 = ty_i * TR;
                for (int c = 0; c < p.C; ++c, ++it) {
                    const int s = it % S;
                    const uint32_t ph = (it / S) & 1u;
                    if (it >= (uint32_t)S) tma::wait_parity(&empty[s], ph ^ 1u, abort_flag, p.status, 1);
                    tma::mbar_arrive_expect_tx(&full[s], (uint32_t)(STAGE * 4));
                    float *stage = ring + s * STAGE;
                    if (ND == 3) {
                        if (DO_K) tma::tensor_g2s_5d(stage, &map_in, x0, y0, z, c, n, &full[s]);
                        if (DO_X) tma::tensor_g2s_5d(stage + (DO_K ? TR * TX : 0), &map_gin, x0, y0, z, c, n, &full[s]);
                    } else {
                        if (DO_K) tma::tensor_g2s_4d(stage, &map_in, x0, y0, c, n, &full[s]);
                        if (DO_X) tma::tensor_g2s_4d(stage + (DO_K ? TR * TX : 0), &map_gin, x0, y0, c, n, &full[s]);
                    }
                }
            }
        }
        return;  // every box this warp requested is awaited by the consumers below
    }

    // -------------------------------- consumer warps --------------------------------
    const int xq = tid % TXQ, rpass = tid / TXQ;
    uint32_t it = 0;
    float bsum = 0.f;
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        const int tx_i = (int)(tile % p.tiles_x);
        const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
        const long long nz = tile / tiles_per_plane;
        const int z = (int)(nz % p.Z), n = (int)(nz / p.Z);
        const int x0 = tx_i * TX, y0 = ty_i * TR;

        // ---- stage the folded rows of m for the RT row taps of this tile ----
        tma::named_barrier(1, kConsumers);  // the previous tile's reads of `rows` are done
        const float *go_n = p.gout + n * p.go_sn;
        const float *out_n = p.out ? p.out + n * p.out_sn : nullptr;
        const int quads = TXP / 4;
        // Each warp stages RT*TR/8 rows, three at a time so that six independent 128-bit
        // global loads are in flight per thread.
        constexpr int ROWS_PER_WARP = RT * TR / kConsumerWarps;
        constexpr int U = 3;
        static_assert(ROWS_PER_WARP % U == 0, "rows per warp must be a multiple of the batch");
        for (int rb = 0; rb < ROWS_PER_WARP; rb += U) {
            int zs[U][2], ys[U][2], nzs[U], nys[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int rowid = warp + kConsumerWarps * (rb + u);
                const int rt = rowid / TR, r = rowid - rt * TR;
                const int y = y0 + r;
                nys[u] = 0;
                if (ND == 3) {
                    nzs[u] = adjoint_sources_dev(z, rt / 3, p.d, p.Z, zs[u]);
                } else {
                    nzs[u] = 1;
                    zs[u][0] = 0;
                }
                if (y < p.Y) nys[u] = adjoint_sources_dev(y, (ND == 3) ? rt % 3 : rt, p.d, p.Y, ys[u]);
                if (nzs[u] == 0) nys[u] = 0;
            }
            for (int q4 = lane; q4 < quads; q4 += 32) {
                const int px = x0 - p.Dp + 4 * q4;
                const bool inside = px >= 0 && px < p.X;
                float4 g[U], o[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    g[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    o[u] = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (inside && nys[u] > 0) {
                        g[u] = ld4(go_n + zs[u][0] * p.go_sz + (int64_t)ys[u][0] * p.go_sy + px);
                        if (out_n) o[u] = ld4(out_n + zs[u][0] * p.out_sz + (int64_t)ys[u][0] * p.out_sy + px);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    float4 acc;
                    acc.x = o[u].x > 0.f ? g[u].x : 0.f;
                    acc.y = o[u].y > 0.f ? g[u].y : 0.f;
                    acc.z = o[u].z > 0.f ? g[u].z : 0.f;
                    acc.w = o[u].w > 0.f ? g[u].w : 0.f;
                    if (inside && nzs[u] * nys[u] > 1) {  // folded sources: border rows only
                        for (int a = 0; a < nzs[u]; ++a)
                            for (int b = (a == 0 ? 1 : 0); b < nys[u]; ++b) {
                                float4 g2 = ld4(go_n + zs[u][a] * p.go_sz + (int64_t)ys[u][b] * p.go_sy + px);
                                if (out_n) {
                                    const float4 o2 = ld4(out_n + zs[u][a] * p.out_sz + (int64_t)ys[u][b] * p.out_sy + px);
                                    g2.x = o2.x > 0.f ? g2.x : 0.f;
                                    g2.y = o2.y > 0.f ? g2.y : 0.f;
                                    g2.z = o2.z > 0.f ? g2.z : 0.f;
                                    g2.w = o2.w > 0.f ? g2.w : 0.f;
                                }
                                acc.x += g2.x, acc.y += g2.y, acc.z += g2.z, acc.w += g2.w;
                            }
                    }
                    const int rowid = warp + kConsumerWarps * (rb + u);
                    *reinterpret_cast<float4 *>(rows + (int64_t)rowid * TXP + 4 * q4) = acc;
                }
            }
        }
        tma::named_barrier(1, kConsumers);

        // ---- per-thread M_t for its P voxels ----
        float M[TAPS][P];
        bool valid[J];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int r = rpass + RPP * j;
            valid[j] = (y0 + r) < p.Y && (x0 + 4 * xq) < p.X;
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                const float *row = rows + (int64_t)(rt * TR + r) * TXP + p.Dp;  // row[i] <-> image x = x0 + i
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = 4 * xq + e;
                    const int q = x0 + i;
                    float m0 = row[i + p.d];
                    float m2 = row[i - p.d];
                    if (q < p.X) {
                        if (q <= p.d - 1) m0 += row[p.d - 1 - q - x0];
                        if (q >= p.X - p.d) m2 += row[2 * p.X - 1 - q - p.d - x0];
                    }
                    M[rt * 3 + 0][j * 4 + e] = m0;
                    M[rt * 3 + 1][j * 4 + e] = row[i];
                    M[rt * 3 + 2][j * 4 + e] = m2;
                }
            }
            if (valid[j]) {
#pragma unroll
                for (int e = 0; e < 4; ++e) bsum += M[(RT / 2) * 3 + 1][j * 4 + e];
            }
        }

        float *gi_tile = DO_X ? p.gin + n * p.gi_sn + z * p.gi_sz + (int64_t)y0 * p.gi_sy + x0 + 4 * xq : nullptr;

        // ---- stream the C input channels past the registers ----
        for (int c = 0; c < p.C; ++c, ++it) {
            const int s = it % S;
            tma::wait_parity(&full[s], (it / S) & 1u, abort_flag, p.status, 2);
            const float *stage = ring + s * STAGE;
            float4 a[J], g[J];
#pragma unroll
            for (int j = 0; j < J; ++j) {
                const int idx = (rpass + RPP * j) * TX + 4 * xq;
                if (DO_K) a[j] = ld4(stage + idx);  // zero outside the image (TMA fill)
                if (DO_X) g[j] = ld4(stage + (DO_K ? TR * TX : 0) + idx);
            }
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&empty[s]);

            if (DO_X) {
                float w[TAPS_PAD];
                const float4 *wp = reinterpret_cast<const float4 *>(wsm + c * TAPS_PAD);
#pragma unroll
                for (int i = 0; i < TAPS_PAD / 4; ++i) {
                    const float4 t4 = wp[i];
                    w[4 * i + 0] = t4.x, w[4 * i + 1] = t4.y, w[4 * i + 2] = t4.z, w[4 * i + 3] = t4.w;
                }
                const bool live = !*abort_flag;
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    float gv[4] = {g[j].x, g[j].y, g[j].z, g[j].w};
#pragma unroll
                    for (int t = 0; t < TAPS; ++t)
#pragma unroll
                        for (int e = 0; e < 4; ++e) gv[e] = fmaf(w[t], M[t][j * 4 + e], gv[e]);
                    if (valid[j] && live)
                        *reinterpret_cast<float4 *>(gi_tile + c * p.gi_sc + (int64_t)(rpass + RPP * j) * p.gi_sy) =
                            make_float4(gv[0], gv[1], gv[2], gv[3]);
                }
            }
            if (DO_K) {
                float acc[NV];
#pragma unroll
                for (int t = 0; t < NV; ++t) {
                    float s_ = 0.f;
                    if (t < TAPS) {
#pragma unroll
                        for (int j = 0; j < J; ++j) {
                            s_ = fmaf(a[j].x, M[t][j * 4 + 0], s_);
                            s_ = fmaf(a[j].y, M[t][j * 4 + 1], s_);
                            s_ = fmaf(a[j].z, M[t][j * 4 + 2], s_);
                            s_ = fmaf(a[j].w, M[t][j * 4 + 3], s_);
                        }
                    }
                    acc[t] = s_;
                }
                const float tot = warp_reduce_scatter<NV>(acc, lane);
                if (lane < TAPS) wacc[(warp * p.C + c) * TAPS_PAD + lane] += tot;
            }
        }
    }

    // ---- block epilogue: fixed-order sums of the warp slots, one partial per block ----
    tma::named_barrier(1, kConsumers);
    const bool live = !*abort_flag;
    if (DO_K && live) {
        float *dst = p.part_k + (int64_t)blockIdx.x * p.C * TAPS;
        for (int i = tid; i < p.C * TAPS; i += kConsumers) {
            const int c = i / TAPS, t = i - c * TAPS;
            float s_ = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) s_ += wacc[(w * p.C + c) * TAPS_PAD + t];
            dst[i] = s_;
        }
    }
    if (p.part_b) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) bsum += __shfl_down_sync(0xffffffffu, bsum, off);
        if (lane == 0) red[warp] = bsum;
        tma::named_barrier(1, kConsumers);
        if (tid == 0 && live) {
            float s_ = 0.f;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) s_ += red[w];
            p.part_b[blockIdx.x] = s_;
        }
    }
}

// Host-side launcher of one instantiation; defined in fast_backward_impl.cuh.
typedef int (*BwdLaunchFn)(const CUtensorMap &, const CUtensorMap &, const BwdParams &, int grid, size_t smem, cudaStream_t);

}  // namespace fast
}  // namespace msd

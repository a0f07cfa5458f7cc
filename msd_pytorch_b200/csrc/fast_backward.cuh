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
// gin[c] straight from registers with 128-bit global stores.  The halo rows of gout and
// out that the NEXT tile's M_t need (3 or 9 row-shifted boxes each, out-of-image parts
// zero-filled) are TMA loads as well, issued one tile ahead into their own buffer, so no
// thread ever waits for a plain global load on the critical path.  Blocks are persistent
// and take tiles in a fixed round-robin order.
//
// Weight gradient reduction (deterministic, two passes): per channel each warp sums its
// threads' 9 (27) partials with a shuffle reduce-scatter and adds them to its own slot in
// shared memory; at the end of the block the eight warp slots are added in warp order and
// written to `part_k[block]`; a second kernel adds the blocks' partials in block order.
#pragma once
#include <type_traits>
#include "common.cuh"
#include "kernels.h"
#include "tma.cuh"

namespace msd {
namespace fast {

// Consumer warps per block (+ one producer warp).  Registers are allocated per four warps:
// 8 + 1 and 11 + 1 warps both leave 168 registers per thread, so the register-hungry 3D
// kernel runs 11 consumer warps; 2D keeps 8 (its 16-row tiles divide the benchmark images).
constexpr int bwd_consumer_warps(int nd) { return nd == 3 ? 11 : 8; }
constexpr int kMaxConsumerWarps = 11;
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
    int z0, ZW;  // planes [z0, z0 + ZW) are processed (the whole volume unless a z-slab window is set)
    int d, Dp;  // dilation and dilation rounded up to a multiple of 4
    int tiles_x, tiles_y;
    long long num_tiles;
    int stages;
    int mask_channel;  // input channel whose new gradient is stored already gated by in[c] > 0 (-1: none)
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

// The same for CU independent vectors at once (their shuffle chains interleave).
template <int NV, int CU>
__device__ __forceinline__ void warp_reduce_scatter_multi(float (&v)[CU][NV], int lane, float (&out)[CU]) {
#pragma unroll
    for (int h = NV / 2; h >= 1; h >>= 1) {
        const bool up = (lane & h) != 0;
#pragma unroll
        for (int i = 0; i < h; ++i)
#pragma unroll
            for (int u = 0; u < CU; ++u) {
                const float send = up ? v[u][i] : v[u][i + h];
                const float keep = up ? v[u][i + h] : v[u][i];
                v[u][i] = keep + __shfl_xor_sync(0xffffffffu, send, h);
            }
    }
#pragma unroll
    for (int u = 0; u < CU; ++u) {
        float r = v[u][0];
        if (NV == 16) r += __shfl_xor_sync(0xffffffffu, r, 16);
        out[u] = r;
    }
}

// Channels processed per loop iteration.
template <int ND, int J>
struct BwdUnroll {
    static constexpr int kChannels = (ND == 2) ? 2 : 1;
};

__device__ __forceinline__ float4 ld4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// Blocks per SM the kernel is compiled for: the 4-voxel-per-thread 2D variant is small
// enough for two resident blocks, so that one block's tile set-up overlaps the other's streaming.
template <int ND, int J>
struct BwdOccupancy {
    static constexpr int kBlocksPerSM = (ND == 2 && J == 1) ? 2 : 1;
};

template <int ND, int TXQ, int J, bool DO_X, bool DO_K>
__global__ void __launch_bounds__(bwd_consumer_warps(ND) * 32 + 32, BwdOccupancy<ND, J>::kBlocksPerSM)
fused_backward_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_gin,
                      const __grid_constant__ CUtensorMap map_gout, const __grid_constant__ CUtensorMap map_out, const BwdParams p) {
    using T = BwdTraits<ND>;
    constexpr int RT = T::RT, TAPS = T::TAPS, TAPS_PAD = T::TAPS_PAD, NV = T::NV;
    constexpr int kConsumerWarps = bwd_consumer_warps(ND), kConsumers = kConsumerWarps * 32, kBwdThreads = kConsumers + 32;
    constexpr int TX = TXQ * 4;
    constexpr int RPP = kConsumers / TXQ;  // rows per pass
    constexpr int TR = RPP * J;            // rows per tile
    constexpr int P = 4 * J;               // voxels per thread
    constexpr int NARR = (DO_X ? 1 : 0) + (DO_K ? 1 : 0);
    constexpr int STAGE = NARR * TR * TX;  // floats per ring stage

    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t *empty = full + kMaxStages;
    uint64_t *halo_full = empty + kMaxStages;  // the halo rows of a tile have landed
    uint64_t *halo_empty = halo_full + 1;      // all consumer warps are done with them
    volatile int *abort_flag = reinterpret_cast<volatile int *>(halo_empty + 1);
    float *red = reinterpret_cast<float *>(smem_raw + 192);  // 16 floats
    const int TXP = TX + 2 * p.Dp;
    const bool gate = p.out != nullptr;
    // TMA destinations first (128-byte aligned): halo rows of gout (turned into the folded
    // rows of m in place), halo rows of out, then the ring.
    float *rows = reinterpret_cast<float *>(smem_raw + 256);
    // each of the RT halo boxes gets a slot rounded up to 128 bytes (TMA destinations)
    const int HSLOT = (TR * TXP + 31) & ~31;
    const int halo_floats = RT * HSLOT;
    float *orows = rows + halo_floats;
    float *ring = orows + (gate ? halo_floats : 0);
    float *wsm = ring + (size_t)p.stages * STAGE;
    float *wacc = wsm + (DO_X ? p.C * TAPS_PAD : 0);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            tma::mbar_init(&full[s], 1);
            tma::mbar_init(&empty[s], kConsumerWarps);
        }
        tma::mbar_init(halo_full, 1);
        tma::mbar_init(halo_empty, kConsumerWarps);
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
    tma::allow_dependents();
    __syncthreads();
    // everything above only touched this layer's constants; the gradient channels below were
    // written by the kernel of the layer above
    tma::grid_dependency_wait();

    const long long tiles_per_plane = (long long)p.tiles_x * p.tiles_y;

    if (warp == kConsumerWarps) {
        // ------------------------------ producer warp ------------------------------
        // One tiled TMA load per array and channel: the TR x TX tile of in[c] and of gin[c].
        // Parts of the box beyond the image are zero-filled by the TMA unit.
        if (lane == 0) {
            if (DO_K) tma::prefetch_tensormap(&map_in);
            if (DO_X) tma::prefetch_tensormap(&map_gin);
            tma::prefetch_tensormap(&map_gout);
            if (gate) tma::prefetch_tensormap(&map_out);
            const uint32_t halo_bytes = (uint32_t)(RT * TR * TXP * 4) * (gate ? 2u : 1u);
            // Halo rows of one tile: row tap (tz, ty) reads the rows shifted by d (1 - t).
            auto issue_halo = [&](long long tile) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const long long nz = tile / tiles_per_plane;
                const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
                const int bx = tx_i * TX - p.Dp, y0 = ty_i * TR;
                tma::mbar_arrive_expect_tx(halo_full, halo_bytes);
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    const int ty = (ND == 3) ? rt % 3 : rt, tz = (ND == 3) ? rt / 3 : 1;
                    const int by = y0 + p.d * (1 - ty), bz = z + p.d * (1 - tz);
                    float *dg = rows + rt * HSLOT, *dout = orows + rt * HSLOT;
                    if (ND == 3) {
                        tma::tensor_g2s_5d(dg, &map_gout, bx, by, bz, 0, n, halo_full);
                        if (gate) tma::tensor_g2s_5d(dout, &map_out, bx, by, bz, 0, n, halo_full);
                    } else {
                        tma::tensor_g2s_4d(dg, &map_gout, bx, by, 0, n, halo_full);
                        if (gate) tma::tensor_g2s_4d(dout, &map_out, bx, by, 0, n, halo_full);
                    }
                }
            };
            uint32_t it = 0, tcount = 0;
            if ((long long)blockIdx.x < p.num_tiles) issue_halo(blockIdx.x);
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tcount) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const long long nz = tile / tiles_per_plane;
                const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
                const int x0 = tx_i * TX, y0 = ty_i * TR;
                // The next tile's halo rows go out once this tile's first `S` channels are
                // requested: by then the ring is what the producer waits on anyway.
                const int halo_at = (p.C < S ? p.C : S) - 1;
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
                    if (c == halo_at && tile + gridDim.x < p.num_tiles) {
                        tma::wait_parity(halo_empty, tcount & 1u, abort_flag, p.status, 5);
                        issue_halo(tile + gridDim.x);
                    }
                }
            }
        }
        return;  // every box this warp requested is awaited by the consumers below
    }

    // -------------------------------- consumer warps --------------------------------
    const int xq = tid % TXQ, rpass = tid / TXQ;
    uint32_t it = 0, tcount = 0;
    float bsum = 0.f;
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tcount) {
        const int tx_i = (int)(tile % p.tiles_x);
        const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
        const long long nz = tile / tiles_per_plane;
        const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
        const int x0 = tx_i * TX, y0 = ty_i * TR;

        // ---- turn the halo rows (landed by TMA) into the folded rows of m, in place ----
        tma::wait_parity(halo_full, tcount & 1u, abort_flag, p.status, 6);
        const float *go_n = p.gout + n * p.go_sn;
        const float *out_n = gate ? p.out + n * p.out_sn : nullptr;
        const int quads = TXP / 4;
        // Rows within d of a y (z) border also collect a mirrored source row; those few are
        // fetched with plain loads.
        const bool fold_rows = (y0 < p.d) || (y0 + TR + p.d > p.Y) || (ND == 3 && (z < p.d || z + p.d >= p.Z));
        // (with an already gated gradient and no border rows the boxes are final as they landed:
        // no pass over them and no barrier - both conditions are uniform over the block)
        const bool touch_rows = gate || fold_rows;
        for (int item = tid; touch_rows && item < RT * TR * quads; item += kConsumers) {
            const int rowid = item / quads, q4 = item - rowid * quads;
            const int rt_ = rowid / TR;
            const int soff = rt_ * HSLOT + (rowid - rt_ * TR) * TXP + 4 * q4;  // slot of the row tap + row inside it
            float4 g = *reinterpret_cast<const float4 *>(rows + soff);
            if (gate) {
                const float4 o = *reinterpret_cast<const float4 *>(orows + soff);
                g.x = o.x > 0.f ? g.x : 0.f;
                g.y = o.y > 0.f ? g.y : 0.f;
                g.z = o.z > 0.f ? g.z : 0.f;
                g.w = o.w > 0.f ? g.w : 0.f;
            }
            if (fold_rows) {
                const int rt = rowid / TR, r = rowid - rt * TR;
                const int y = y0 + r, px = x0 - p.Dp + 4 * q4;
                int zs[2], ys[2], nzs = 1, nys = 0;
                zs[0] = 0;
                if (ND == 3) nzs = adjoint_sources_dev(z, rt / 3, p.d, p.Z, zs);
                if (y < p.Y && nzs > 0) nys = adjoint_sources_dev(y, (ND == 3) ? rt % 3 : rt, p.d, p.Y, ys);
                if (px >= 0 && px < p.X && nzs * nys > 0) {
                    // The TMA box holds the direct source (zero when it lies outside); add the
                    // others.  The direct source is the first entry exactly when it is inside.
                    const int dy = y - p.d * (((ND == 3) ? rt % 3 : rt) - 1);
                    const int dz = (ND == 3) ? z - p.d * (rt / 3 - 1) : 0;
                    for (int a = 0; a < nzs; ++a)
                        for (int b = 0; b < nys; ++b) {
                            if (ys[b] == dy && (ND != 3 || zs[a] == dz)) continue;  // already there
                            float4 g2 = ld4(go_n + zs[a] * p.go_sz + (int64_t)ys[b] * p.go_sy + px);
                            if (out_n) {
                                const float4 o2 = ld4(out_n + zs[a] * p.out_sz + (int64_t)ys[b] * p.out_sy + px);
                                g2.x = o2.x > 0.f ? g2.x : 0.f;
                                g2.y = o2.y > 0.f ? g2.y : 0.f;
                                g2.z = o2.z > 0.f ? g2.z : 0.f;
                                g2.w = o2.w > 0.f ? g2.w : 0.f;
                            }
                            g.x += g2.x, g.y += g2.y, g.z += g2.z, g.w += g2.w;
                        }
                }
            }
            *reinterpret_cast<float4 *>(rows + soff) = g;
        }
        if (touch_rows) tma::named_barrier(1, kConsumers);

        // ---- per-thread M_t for its P voxels ----
        float M[TAPS][P];
        bool valid[J];
        const bool fold_x = (x0 < p.d) || (x0 + TX + p.d > p.X);
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int r = rpass + RPP * j;
            valid[j] = (y0 + r) < p.Y && (x0 + 4 * xq) < p.X;
#pragma unroll
            for (int rt = 0; rt < RT; ++rt) {
                const float *row = rows + rt * HSLOT + r * TXP + p.Dp;  // row[i] <-> image x = x0 + i
                const float4 ctr = *reinterpret_cast<const float4 *>(row + 4 * xq);
                const float cv[4] = {ctr.x, ctr.y, ctr.z, ctr.w};
                // The x-taps need the 4 consecutive values that start d to the right / left of
                // the thread's own quad: two aligned 128-bit loads each and a shift by d mod 4
                // (warp-uniform) instead of four 4-way bank-conflicted scalar loads.
                const int sh = p.d & 3, qd = p.d >> 2;
                const float4 *row4 = reinterpret_cast<const float4 *>(row);
                float up[8], dn[8];
                {
                    const float4 l0 = row4[xq + qd], l1 = sh ? row4[xq + qd + 1] : l0;
                    up[0] = l0.x, up[1] = l0.y, up[2] = l0.z, up[3] = l0.w, up[4] = l1.x, up[5] = l1.y, up[6] = l1.z, up[7] = l1.w;
                    // values [4xq - d, 4xq - d + 4): quad xq - qd - (sh ? 1 : 0), offset (4 - sh) & 3
                    const float4 r0 = row4[xq - qd - (sh ? 1 : 0)], r1 = sh ? row4[xq - qd] : r0;
                    dn[0] = r0.x, dn[1] = r0.y, dn[2] = r0.z, dn[3] = r0.w, dn[4] = r1.x, dn[5] = r1.y, dn[6] = r1.z, dn[7] = r1.w;
                }
                float m0v[4], m2v[4];
                switch (sh) {
                    case 0:
#pragma unroll
                        for (int e = 0; e < 4; ++e) m0v[e] = up[e], m2v[e] = dn[e];
                        break;
                    case 1:
#pragma unroll
                        for (int e = 0; e < 4; ++e) m0v[e] = up[e + 1], m2v[e] = dn[e + 3];
                        break;
                    case 2:
#pragma unroll
                        for (int e = 0; e < 4; ++e) m0v[e] = up[e + 2], m2v[e] = dn[e + 2];
                        break;
                    default:
#pragma unroll
                        for (int e = 0; e < 4; ++e) m0v[e] = up[e + 3], m2v[e] = dn[e + 1];
                        break;
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = 4 * xq + e;
                    float m0 = m0v[e];
                    float m2 = m2v[e];
                    if (fold_x) {  // block-uniform: only tiles next to the left / right border
                        const int q = x0 + i;
                        // only the few lanes within d of the border load (a load by all lanes
                        // with a stride of four floats costs four shared-memory wavefronts)
                        const bool f0 = q < p.X && q <= p.d - 1, f2 = q < p.X && q >= p.X - p.d;
                        if (f0) m0 += row[p.d - 1 - q - x0];
                        if (f2) m2 += row[2 * p.X - 1 - q - p.d - x0];
                    }
                    M[rt * 3 + 0][j * 4 + e] = m0;
                    M[rt * 3 + 1][j * 4 + e] = cv[e];
                    M[rt * 3 + 2][j * 4 + e] = m2;
                }
            }
            if (valid[j]) {
#pragma unroll
                for (int e = 0; e < 4; ++e) bsum += M[(RT / 2) * 3 + 1][j * 4 + e];
            }
        }
        // this warp no longer needs the halo rows: the producer may load the next tile's
        // (the fence orders this thread's shared-memory accesses before the TMA writes)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(halo_empty);

        float *gi_tile = DO_X ? p.gin + n * p.gi_sn + z * p.gi_sz + (int64_t)y0 * p.gi_sy + x0 + 4 * xq : nullptr;

        // ---- stream the C input channels past the registers ----
        // CU channels are processed per iteration so that their FMA blocks and shuffle
        // reduce-scatters (long dependent chains) interleave.
        auto body = [&](auto cu_tag, int c) {
            constexpr int CU = decltype(cu_tag)::value;
            float4 a[CU][J], g[CU][J];
#pragma unroll
            for (int u = 0; u < CU; ++u) {
                const int s = (it + u) % S;
                tma::wait_parity(&full[s], ((it + u) / S) & 1u, abort_flag, p.status, 2);
                const float *stage = ring + s * STAGE;
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    const int idx = (rpass + RPP * j) * TX + 4 * xq;
                    if (DO_K) a[u][j] = ld4(stage + idx);  // zero outside the image (TMA fill)
                    if (DO_X) g[u][j] = ld4(stage + (DO_K ? TR * TX : 0) + idx);
                }
            }
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int u = 0; u < CU; ++u) tma::mbar_arrive(&empty[(it + u) % S]);
            }
            it += CU;

            if (DO_K) {
                float acc[CU][NV];
#pragma unroll
                for (int u = 0; u < CU; ++u)
#pragma unroll
                    for (int t = 0; t < NV; ++t) {
                        float s_ = 0.f;
                        if (t < TAPS) {
#pragma unroll
                            for (int j = 0; j < J; ++j) {
                                s_ = fmaf(a[u][j].x, M[t][j * 4 + 0], s_);
                                s_ = fmaf(a[u][j].y, M[t][j * 4 + 1], s_);
                                s_ = fmaf(a[u][j].z, M[t][j * 4 + 2], s_);
                                s_ = fmaf(a[u][j].w, M[t][j * 4 + 3], s_);
                            }
                        }
                        acc[u][t] = s_;
                    }
                float tot[CU];
                warp_reduce_scatter_multi<NV, CU>(acc, lane, tot);
                if (lane < TAPS) {
#pragma unroll
                    for (int u = 0; u < CU; ++u) wacc[(warp * p.C + c + u) * TAPS_PAD + lane] += tot[u];
                }
            }
            if (DO_X) {
                const bool live = !*abort_flag;
#pragma unroll
                for (int u = 0; u < CU; ++u) {
                    float w[TAPS_PAD];
                    const float4 *wp = reinterpret_cast<const float4 *>(wsm + (c + u) * TAPS_PAD);
#pragma unroll
                    for (int i = 0; i < TAPS_PAD / 4; ++i) {
                        const float4 t4 = wp[i];
                        w[4 * i + 0] = t4.x, w[4 * i + 1] = t4.y, w[4 * i + 2] = t4.z, w[4 * i + 3] = t4.w;
                    }
#pragma unroll
                    for (int j = 0; j < J; ++j) {
                        float gv[4] = {g[u][j].x, g[u][j].y, g[u][j].z, g[u][j].w};
#pragma unroll
                        for (int t = 0; t < TAPS; ++t)
#pragma unroll
                            for (int e = 0; e < 4; ++e) gv[e] = fmaf(w[t], M[t][j * 4 + e], gv[e]);
                        if (DO_K && (c + u) == p.mask_channel) {
                            // this channel is the output of the layer below: hand its gradient
                            // over already multiplied by that layer's ReLU gate
                            gv[0] = a[u][j].x > 0.f ? gv[0] : 0.f;
                            gv[1] = a[u][j].y > 0.f ? gv[1] : 0.f;
                            gv[2] = a[u][j].z > 0.f ? gv[2] : 0.f;
                            gv[3] = a[u][j].w > 0.f ? gv[3] : 0.f;
                        }
                        if (valid[j] && live)
                            *reinterpret_cast<float4 *>(gi_tile + (c + u) * p.gi_sc + (int64_t)(rpass + RPP * j) * p.gi_sy) =
                                make_float4(gv[0], gv[1], gv[2], gv[3]);
                    }
                }
            }
        };
        {
            constexpr int CUMAX = BwdUnroll<ND, J>::kChannels;
            int c = 0;
            for (; c + CUMAX <= p.C; c += CUMAX) body(std::integral_constant<int, CUMAX>{}, c);
            for (; c < p.C; ++c) body(std::integral_constant<int, 1>{}, c);
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

// Host-side launcher of one instantiation (defined in fast_backward_2d.cu / fast_backward_3d.cu).
typedef int (*BwdLaunchFn)(const CUtensorMap *maps, const BwdParams &, int grid, size_t smem, cudaStream_t);  // maps: in, gin, gout, out

}  // namespace fast
}  // namespace msd

// Fused backward of one MSD layer (one output channel, float32; 3D and 2D) with the consumer
// warps split by role.  Same mathematics and buffers as fused_backward_kernel
// (fast_backward.cuh); what differs is who computes what:
//
//   X warps  voxels across lanes (4 consecutive x per thread), the 27 (9) values M_t of each
//            voxel in registers: per channel 27 (9) x 4 FMAs update the input gradient, one
//            128-bit store.  No reduction of any kind.
//   K warps  3D: lane = (quarter-warp, tap lane): each lane keeps M_t[v] for 4 taps (tap lane + 8 a)
//            and 16 voxels of half a tile row in registers, reads in[c][v] with 128-bit
//            shared loads and accumulates  sum_v in[c][v] * M_t[v]  with packed FMAs; the
//            four quarter-warps' sums meet in a 3-shuffle reduce-scatter (the full shuffle
//            tree of the unsplit kernel costs 124 instructions per 216 FMAs in 3D).
//            2D: a lane keeps tap `tap lane` (0..7) for the 32 voxels of its quarter of a tile
//            row and the ninth tap for four of them (the eight tap lanes of a quarter-warp share
//            it out); five shuffles per channel.
//
// A tile is 4 rows x 128 columns of one z-plane (3D) or 8 rows x 128 columns (2D).  The block
// has four warpgroups:
//   warps 0-3    X warps, one per tile row (2D: rows w and w + 4)   (registers raised to kSplitRegsX)
//   warps 4-11   K warps, 3D: (row, half) = (w-4)/2, (w-4)%2; 2D: row w-4  (the launch's 128 registers)
//   warp 12      TMA producer                            (registers lowered to kSplitRegsP)
//   warps 13-15  builders of the table of M (below)      (same warpgroup as the producer)
// so that each of the four warp schedulers (warp id mod 4) carries one X warp and two K warps.
// The register file is re-divided between the warpgroups with setmaxnreg: the 3D X warps need
// 108 registers for M alone, the producer and the builders few.
//
// Data movement.  One ring stage holds 4 (2D: 2) consecutive channels of the tile: two TMA
// boxes (activations, gradients) of 4 x 4 x 128 (2 x 8 x 128) floats, so that the cost of issuing a
// copy and of the full/empty hand-shake is paid once per kSplitCB channels.  The 9 (3) halo row
// groups of gout (and of out, for the ReLU gate) land by TMA in one of two buffers (tiles
// alternate), requested a whole tile ahead.  The builder warps turn them into
// the table  Msm[t][row][x] = M_t(voxel)  in two short passes (gate + y/z folds in place; x
// shifts + x folds into the table) while the consumers are still streaming the channels of
// the previous tile; both kinds of consumer warps then fill their registers from the table
// with aligned 128-bit loads and no arithmetic - the per-tile set-up never holds the channel
// stream up.  The table's tap stride is 4 mod 32 banks, which makes the K warps' lane-per-tap
// loads conflict-free.  Hand-shakes: halo_full (producer -> builders), halo_empty (builders ->
// producer), table_full (builders -> consumers), m_done (consumers -> builders: the table may
// be overwritten).
//
// Requirements (checked by the host): X a multiple of 128, dilation <= 12, both gradients wanted.
#pragma once
#include "fast_backward.cuh"

namespace msd {
namespace fast {

constexpr int kSplitRows = 4;                                     // 3D: rows per tile
constexpr int split_rows(int nd) { return nd == 3 ? kSplitRows : 8; }  // 2D: 8 rows (two per X warp, one per K warp)
constexpr int kSplitTX = 128;
constexpr int kSplitCB = 4;                                       // 3D: channels per ring stage
constexpr int split_cb(int nd) { return nd == 3 ? kSplitCB : 2; }  // 2D: two (a stage is 2 tensors x 2 channels x 8 rows x 128)
constexpr int kSplitKU = 2;                                       // channels a K warp processes per loop iteration (4: measured 4 % slower)
constexpr int kSplitKHalf = 64;                                   // 3D: voxels per K warp (half a row); 2D: a whole row
constexpr int kSplitXWarps = 4;
constexpr int kSplitKWarps = 8;
constexpr int kSplitConsumerWarps = kSplitXWarps + kSplitKWarps;  // 12
constexpr int kSplitConsumers = kSplitConsumerWarps * 32;         // 384
constexpr int kSplitThreads = 512;                                // four warpgroups
constexpr int split_taps_pad(int nd) { return nd == 3 ? 28 : 12; }  // floats per channel of weights / per (K warp, channel) slot in shared memory
constexpr int kSplitMaxD = 12;                                    // border columns handled per side
constexpr int kSplitMaxStages = 8;
constexpr int kSplitHeaderBytes = 512;                            // barriers, abort flag, bias slots
constexpr int kSplitBuilderWarps = 3;                             // warps 13-15
constexpr int kSplitBuilders = kSplitBuilderWarps * 32;
constexpr int kSplitRegsX = 176, kSplitRegsP = 80;  // 128 x 176 + 256 x 128 + 128 x 80 = 65536 registers

// Bounded wait with a fast path: one try_wait before the generic bounded loop.
__device__ __forceinline__ void split_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int code) {
    if (tma::mbar_try_wait(bar, parity)) return;
    tma::wait_parity(bar, parity, abort_flag, status, code);
}

// Pass A: turns the halo rows of one tile (landed by TMA in `rows` / `orows`, slots of HSLOT
// floats) into the rows of m, in place: ReLU gate, plus the mirrored y / z sources next to
// the volume's borders.  Cooperative over the kSplitBuilders builder threads (index btid); the
// caller synchronises them afterwards.
template <int NTHREADS = kSplitBuilders, int TR = kSplitRows, int ND = 3>
__device__ __forceinline__ void split_fill_rows(const BwdParams &p, float *rows, const float *orows, int HSLOT, int TXP, bool gate, int btid, int n,
                                                int z, int y0, int x0) {
    constexpr int RT = ND == 3 ? 9 : 3;
    const bool fold_rows = (y0 < p.d) || (y0 + TR + p.d > p.Y) || (ND == 3 && (z < p.d || z + p.d >= p.Z));
    if (!gate && !fold_rows) return;
    const float *go_n = p.gout + n * p.go_sn;
    const float *out_n = gate ? p.out + n * p.out_sn : nullptr;
    const int quads = TXP / 4;
#pragma unroll 1
    for (int item = btid; item < RT * TR * quads; item += NTHREADS) {
        const int rowid = item / quads, q4 = item - rowid * quads;
        const int rt = rowid / TR, rr = rowid - rt * TR;
        const int soff = rt * HSLOT + rr * TXP + 4 * q4;
        float4 g = *reinterpret_cast<const float4 *>(rows + soff);
        if (gate) {
            const float4 o = *reinterpret_cast<const float4 *>(orows + soff);
            g.x = o.x > 0.f ? g.x : 0.f;
            g.y = o.y > 0.f ? g.y : 0.f;
            g.z = o.z > 0.f ? g.z : 0.f;
            g.w = o.w > 0.f ? g.w : 0.f;
        }
        if (fold_rows) {
            const int y = y0 + rr, px = x0 - p.Dp + 4 * q4;
            int zs[2], ys[2], nys = 0, nzs = 1;
            zs[0] = 0;
            if (ND == 3) nzs = adjoint_sources_dev(z, rt / 3, p.d, p.Z, zs);
            if (y < p.Y && nzs > 0) nys = adjoint_sources_dev(y, rt % 3, p.d, p.Y, ys);
            if (px >= 0 && px < p.X && nzs * nys > 0) {
                const int dy = y - p.d * (rt % 3 - 1), dz = ND == 3 ? z - p.d * (rt / 3 - 1) : 0;
                for (int a = 0; a < nzs; ++a)
                    for (int b = 0; b < nys; ++b) {
                        if (ys[b] == dy && zs[a] == dz) continue;  // the TMA box already holds it
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
}

// Floats [S, S + 4) of the eight floats (a, b).
template <int S>
__device__ __forceinline__ float4 split_shift4(const float4 &a, const float4 &b) {
    if (S == 0) return a;
    if (S == 1) return make_float4(a.y, a.z, a.w, b.x);
    if (S == 2) return make_float4(a.z, a.w, b.x, b.y);
    return make_float4(a.w, b.x, b.y, b.z);
}

// Pass B: the table  msm[t * TS + row * 128 + i] = M_t at voxel (row, x0 + i),  t = (tz, ty, tx):
// the row of m that tap (tz, ty) reads, shifted by -d (tx - 1) columns, plus the mirrored x
// source next to the left (tx = 0) / right (tx = 2) border of the image.  One (row tap, row)
// per builder warp and step, four consecutive floats per lane: five aligned 128-bit loads
// (three when d is a multiple of 4) give the three x taps, combined by the shift d mod 4
// (SH, uniform over the launch), and three 128-bit stores write them - no branch in the loop.
// The builder warps share their schedulers with three consumer warps each, so what counts is
// how few instructions a row takes (a version with one scalar load and store per float was
// 2 - 4 % slower on layers of 25 and more channels).
template <int SH, int RT, int TR>
__device__ __forceinline__ void split_build_table_sh(const BwdParams &p, const float *rows, float *msm, int HSLOT, int TXP, int TS, int btid, int x0) {
    constexpr int TX = kSplitTX;
    const bool fold_l = x0 == 0, fold_r = x0 + TX == p.X;
    const int lane = btid & 31, qd = p.d >> 2;
    const bool lane_l = fold_l && 4 * lane < p.d, lane_r = fold_r && 4 * lane + 3 >= TX - p.d;
#pragma unroll 2
    for (int item = btid >> 5; item < RT * TR; item += kSplitBuilderWarps) {
        const int rt = item / TR, rr = item - rt * TR;
        const float *row = rows + rt * HSLOT + rr * TXP + p.Dp;  // row[i] <-> image x = x0 + i
        const float4 *row4 = reinterpret_cast<const float4 *>(row);
        const float4 c = row4[lane];
        const float4 u0 = row4[lane + qd];  // floats [4 lane + d, ...): tap tx = 0
        const float4 q0 = SH == 0 ? u0 : split_shift4<SH>(u0, row4[lane + qd + 1]);
        const float4 l1 = row4[lane - qd];  // floats [4 lane - d, ...): tap tx = 2
        const float4 q2 = SH == 0 ? l1 : split_shift4<(4 - SH) & 3>(row4[lane - qd - 1], l1);
        float v0[4] = {q0.x, q0.y, q0.z, q0.w}, v2[4] = {q2.x, q2.y, q2.z, q2.w};
        if (lane_l) {  // columns i <= d - 1 also get the source d - 1 - i
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (4 * lane + e < p.d) v0[e] += row[p.d - 1 - 4 * lane - e];
        }
        if (lane_r) {  // columns i >= X - d also get 2X - 1 - i - d
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (4 * lane + e >= TX - p.d) v2[e] += row[2 * TX - 1 - p.d - 4 * lane - e];
        }
        float *dst = msm + (3 * rt) * TS + rr * TX + 4 * lane;
        *reinterpret_cast<float4 *>(dst) = make_float4(v0[0], v0[1], v0[2], v0[3]);
        *reinterpret_cast<float4 *>(dst + TS) = c;
        *reinterpret_cast<float4 *>(dst + 2 * TS) = make_float4(v2[0], v2[1], v2[2], v2[3]);
    }
}

template <int RT, int TR>
__device__ __forceinline__ void split_build_table(const BwdParams &p, const float *rows, float *msm, int HSLOT, int TXP, int TS, int btid, int x0) {
    switch (p.d & 3) {
        case 0: split_build_table_sh<0, RT, TR>(p, rows, msm, HSLOT, TXP, TS, btid, x0); break;
        case 1: split_build_table_sh<1, RT, TR>(p, rows, msm, HSLOT, TXP, TS, btid, x0); break;
        case 2: split_build_table_sh<2, RT, TR>(p, rows, msm, HSLOT, TXP, TS, btid, x0); break;
        default: split_build_table_sh<3, RT, TR>(p, rows, msm, HSLOT, TXP, TS, btid, x0); break;
    }
}

// One tiled TMA load of a (channels, rows, columns) box: 5-d maps (x, y, z, c, n) in 3D, 4-d maps
// (x, y, c, n) in 2D.
template <int ND>
__device__ __forceinline__ void split_g2s(void *dst, const CUtensorMap *map, int x, int y, int z, int c, int n, uint64_t *bar) {
    if (ND == 3)
        tma::tensor_g2s_5d(dst, map, x, y, z, c, n, bar);
    else
        tma::tensor_g2s_4d(dst, map, x, y, c, n, bar);
}

template <int ND>
__global__ void __launch_bounds__(kSplitThreads, 1)
fused_backward_split_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_gin,
                            const __grid_constant__ CUtensorMap map_gout, const __grid_constant__ CUtensorMap map_out, const BwdParams p) {
    constexpr int RT = ND == 3 ? 9 : 3, TAPS = 3 * RT, WPAD = split_taps_pad(ND);
    constexpr int TX = kSplitTX, TR = split_rows(ND), KH = kSplitKHalf, CB = split_cb(ND);
    constexpr int XR = TR / kSplitXWarps;  // rows per X warp
    constexpr int CHAN = TR * TX;        // floats of one channel of one tensor in a stage
    constexpr int STAGE = 2 * CB * CHAN;  // CB channels of in, then CB channels of gin

    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw);
    uint64_t *empty = full + kSplitMaxStages;
    uint64_t *halo_full = empty + kSplitMaxStages;  // [2] the halo rows of a tile have landed (two buffers, tiles alternate)
    uint64_t *halo_empty = halo_full + 2;           // [2] ... have been turned into the table: the slots are free
    uint64_t *m_done = halo_empty + 2;              // every consumer warp has its M registers: the table is free
    uint64_t *table_full = m_done + 1;              // the table of a tile is complete
    volatile int *abort_flag = reinterpret_cast<volatile int *>(table_full + 1);
    float *red = reinterpret_cast<float *>(smem_raw + 384);
    const int TXP = TX + 2 * p.Dp;
    const bool gate = p.out != nullptr;
    float *rows0 = reinterpret_cast<float *>(smem_raw + kSplitHeaderBytes);
    const int HSLOT = (TR * TXP + 31) & ~31;
    constexpr int TS = TR * TX + 4;  // tap stride of the table: 4 banks apart
    const int HBUF = RT * HSLOT * (gate ? 2 : 1);  // floats of one halo buffer: rows of gout, then (with a gate) rows of out
    float *msm = rows0 + 2 * HBUF;
    float *ring = msm + ((TAPS * TS + 31) & ~31);
    float *wsm = ring + (size_t)p.stages * STAGE;
    float *wacc = wsm + p.C * WPAD;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.stages;
    const int ngroups = (p.C + CB - 1) / CB;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            tma::mbar_init(&full[s], 1);
            tma::mbar_init(&empty[s], kSplitConsumerWarps);
        }
        for (int b = 0; b < 2; ++b) {
            tma::mbar_init(&halo_full[b], 1);
            tma::mbar_init(&halo_empty[b], 1);
        }
        tma::mbar_init(m_done, kSplitConsumerWarps);
        tma::mbar_init(table_full, 1);
        *abort_flag = 0;
        tma::fence_barrier_init();
    }
    for (int i = tid; i < p.C * WPAD; i += kSplitThreads) {
        const int c = i / WPAD, t = i % WPAD;
        wsm[i] = t < TAPS ? p.k[c * TAPS + t] : 0.f;
    }
    for (int i = tid; i < kSplitKWarps * p.C * WPAD; i += kSplitThreads) wacc[i] = 0.f;
    tma::allow_dependents();
    __syncthreads();
    tma::grid_dependency_wait();

    const long long tiles_per_plane = (long long)p.tiles_x * p.tiles_y;

    if (warp >= kSplitConsumerWarps) {
        // ------------------- producer warpgroup: warp 12 issues the copies -------------------
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kSplitRegsP));
        if (warp == kSplitConsumerWarps && lane == 0) {
            tma::prefetch_tensormap(&map_in);
            tma::prefetch_tensormap(&map_gin);
            tma::prefetch_tensormap(&map_gout);
            if (gate) tma::prefetch_tensormap(&map_out);
            const uint32_t halo_bytes = (uint32_t)(RT * TR * TXP * 4) * (gate ? 2u : 1u);
            // Halo rows of the block's `use`-th tile go to buffer use & 1; a buffer is free again once the
            // builders have turned its previous content (tile use - 2) into the table.
            auto issue_halo = [&](long long tile, uint32_t use) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const long long nz = tile / tiles_per_plane;
                const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
                const int bx = tx_i * TX - p.Dp, y0 = ty_i * TR;
                const int b = use & 1;
                float *rows = rows0 + b * HBUF, *orows = rows + RT * HSLOT;
                if (use >= 2) split_wait(&halo_empty[b], ((use >> 1) & 1u) ^ 1u, abort_flag, p.status, 5);
                tma::mbar_arrive_expect_tx(&halo_full[b], halo_bytes);
#pragma unroll 1
                for (int rt = 0; rt < RT; ++rt) {
                    const int by = y0 + p.d * (1 - rt % 3), bz = ND == 3 ? z + p.d * (1 - rt / 3) : 0;
                    split_g2s<ND>(rows + rt * HSLOT, &map_gout, bx, by, bz, 0, n, &halo_full[b]);
                    if (gate) split_g2s<ND>(orows + rt * HSLOT, &map_out, bx, by, bz, 0, n, &halo_full[b]);
                }
            };
            uint32_t it = 0, tcount = 0, s = 0, ph = 0;
            if ((long long)blockIdx.x < p.num_tiles) issue_halo(blockIdx.x, 0);
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tcount) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const long long nz = tile / tiles_per_plane;
                const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
                const int x0 = tx_i * TX, y0 = ty_i * TR;
                for (int g = 0; g < ngroups; ++g, ++it) {
                    if (it >= (uint32_t)S) split_wait(&empty[s], ph ^ 1u, abort_flag, p.status, 1);
                    tma::mbar_arrive_expect_tx(&full[s], (uint32_t)(STAGE * 4));
                    float *stage = ring + s * STAGE;
                    // channels past C are outside the tensor maps: zero-filled, no traffic
                    split_g2s<ND>(stage, &map_in, x0, y0, z, g * CB, n, &full[s]);
                    split_g2s<ND>(stage + CB * CHAN, &map_gin, x0, y0, z, g * CB, n, &full[s]);
                    // the next tile's halo rows go out with this tile's first stage: their buffer was freed
                    // a whole tile ago, so the builders never wait for a request that has not been made
                    if (g == 0 && tile + gridDim.x < p.num_tiles) issue_halo(tile + gridDim.x, tcount + 1);
                    if (++s == (uint32_t)S) s = 0, ph ^= 1u;
                }
            }
        } else if (warp > kSplitConsumerWarps) {
            // ---------------- builder warps: the table of the NEXT tile, while the ----------------
            // ---------------- consumers stream the channels of the current one    ----------------
            const int btid = tid - (kSplitConsumerWarps + 1) * 32;
            uint32_t tcount = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tcount) {
                const int tx_i = (int)(tile % p.tiles_x);
                const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
                const long long nz = tile / tiles_per_plane;
                const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
                const int x0 = tx_i * TX, y0 = ty_i * TR;
                const int hb = tcount & 1;
                float *rows = rows0 + hb * HBUF, *orows = rows + RT * HSLOT;
                split_wait(&halo_full[hb], (tcount >> 1) & 1u, abort_flag, p.status, 6);
                split_fill_rows<kSplitBuilders, TR, ND>(p, rows, orows, HSLOT, TXP, gate, btid, n, z, y0, x0);
                if (tcount) split_wait(m_done, (tcount - 1) & 1u, abort_flag, p.status, 7);  // the previous table has been read
                tma::named_barrier(3, kSplitBuilders);
                split_build_table<RT, TR>(p, rows, msm, HSLOT, TXP, TS, btid, x0);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the reads of the rows, before TMA rewrites them
                tma::named_barrier(3, kSplitBuilders);
                if (btid == 0) {
                    tma::mbar_arrive(&halo_empty[hb]);  // the TMA slots may take the rows of the tile after next
                    tma::mbar_arrive(table_full);
                }
            }
        }
        return;
    }

    uint32_t tcount = 0, s = 0, ph = 0;
    if (warp >= kSplitXWarps) {
        // ===================================== K warps =====================================
        const int kw = warp - kSplitXWarps;
        const int qw = lane >> 3, tl = lane & 7;
        const bool hi = (lane & 16) != 0, mid = (lane & 8) != 0;
        if constexpr (ND == 3) {
        const int r = kw >> 1, h = kw & 1;
        // lane = (qw, tl): taps tl + 8 {0..3}; voxels 4 (4 j + qw) + {0..3}, j = 0..3, of the half row.
        // The four quarter-warps read four neighbouring 16-byte pieces of the activations per
        // load; the eight lanes of a quarter-warp (one phase of a 128-bit shared load) read
        // eight neighbouring taps of the table, whose tap stride of 4 mod 32 banks spreads them
        // over all banks.
        const int tfinal = tl + 8 * ((hi ? 2 : 0) + (mid ? 1 : 0));  // the tap whose sum this lane ends up with
        float *wslot = wacc + (size_t)kw * p.C * WPAD + tfinal;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tcount) {
            split_wait(table_full, tcount & 1u, abort_flag, p.status, 8);

            float2 Mk[4][KH / 8];  // [tap of the lane][pair of neighbouring voxels]: operands of packed FMAs
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const int ta = tl + 8 * a;
                const float4 *m4 = reinterpret_cast<const float4 *>(msm + (ta < TAPS ? ta : 0) * TS + r * TX + KH * h);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float4 q = m4[4 * j + qw];
                    if (ta >= TAPS) q = make_float4(0.f, 0.f, 0.f, 0.f);
                    Mk[a][2 * j] = make_float2(q.x, q.y), Mk[a][2 * j + 1] = make_float2(q.z, q.w);
                }
            }
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(m_done);

            for (int g = 0; g < ngroups; ++g) {
                split_wait(&full[s], ph, abort_flag, p.status, 2);
                const float4 *ain0 = reinterpret_cast<const float4 *>(ring + s * STAGE + r * TX + KH * h) + qw;  // in[g * CB], this half row
                float tot[CB];
                // kSplitKU channels at a time: 4 kSplitKU independent chains of packed FMAs, and one
                // reduce-scatter over the four quarter-warps (fixed tree) for all of them, so that its
                // two shuffle rounds are paid once per group.  The activations are loaded one 16-voxel
                // slice at a time.  Channels past C read a zero-filled stage.
#pragma unroll
                for (int cp = 0; cp < CB; cp += kSplitKU) {
                    const float4 *ain = ain0 + cp * (CHAN / 4);
                    float2 acc[kSplitKU][4];
#pragma unroll
                    for (int u = 0; u < kSplitKU; ++u)
#pragma unroll
                        for (int a = 0; a < 4; ++a) acc[u][a] = make_float2(0.f, 0.f);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float4 av[kSplitKU];
#pragma unroll
                        for (int u = 0; u < kSplitKU; ++u) av[u] = ain[u * (CHAN / 4) + 4 * j];  // one 64-byte run per warp and load
#pragma unroll
                        for (int a = 0; a < 4; ++a)
#pragma unroll
                            for (int u = 0; u < kSplitKU; ++u) acc[u][a] = __ffma2_rn(make_float2(av[u].x, av[u].y), Mk[a][2 * j], acc[u][a]);
#pragma unroll
                        for (int a = 0; a < 4; ++a)
#pragma unroll
                            for (int u = 0; u < kSplitKU; ++u) acc[u][a] = __ffma2_rn(make_float2(av[u].z, av[u].w), Mk[a][2 * j + 1], acc[u][a]);
                    }
                    float k0[kSplitKU], k1[kSplitKU];
#pragma unroll
                    for (int u = 0; u < kSplitKU; ++u) {
                        // sums over the lane's 16 voxels; the lane keeps taps {2 hi, 2 hi + 1} of its four
                        const float s0 = acc[u][0].x + acc[u][0].y, s1 = acc[u][1].x + acc[u][1].y;
                        const float s2 = acc[u][2].x + acc[u][2].y, s3 = acc[u][3].x + acc[u][3].y;
                        k0[u] = (hi ? s2 : s0) + __shfl_xor_sync(0xffffffffu, hi ? s0 : s2, 16);
                        k1[u] = (hi ? s3 : s1) + __shfl_xor_sync(0xffffffffu, hi ? s1 : s3, 16);
                    }
#pragma unroll
                    for (int u = 0; u < kSplitKU; ++u)  // ... then tap 2 hi + mid
                        tot[cp + u] = (mid ? k1[u] : k0[u]) + __shfl_xor_sync(0xffffffffu, mid ? k0[u] : k1[u], 8);
                }
                __syncwarp();
                if (lane == 0) tma::mbar_arrive(&empty[s]);
                if (tfinal < TAPS) {
#pragma unroll
                    for (int cc = 0; cc < CB; ++cc)
                        if (g * CB + cc < p.C) wslot[(g * CB + cc) * WPAD] += tot[cc];
                }
                if (++s == (uint32_t)S) s = 0, ph ^= 1u;
            }
        }
        } else {
        // 2D, nine taps, one K warp per tile row: lane = (qw, tl) keeps tap tl (0..7) for the 32
        // voxels 32 qw + {0..31} of its row and the ninth tap for four of them (the 16-byte piece
        // tl of those 32 voxels), which costs one more 128-bit load (conflict-free: the eight
        // lanes of a phase read 128 consecutive bytes) and two more packed FMAs per channel.
        // Per channel: the sums of tap tl meet over the four quarter-warps, those of tap 8 over
        // all 32 lanes (5 shuffles).
        const int r = kw;
        (void)mid;
        const int tfinal = lane < 8 ? lane : (lane == 16 ? 8 : TAPS);  // the tap whose sum this lane ends up with
        float *wslot = wacc + (size_t)kw * p.C * WPAD + (tfinal < TAPS ? tfinal : 0);
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tcount) {
            split_wait(table_full, tcount & 1u, abort_flag, p.status, 8);

            float2 Mk[16], Mk8[2];  // pairs of neighbouring voxels: operands of packed FMAs
            {
                const float4 *m4 = reinterpret_cast<const float4 *>(msm + tl * TS + r * TX) + 8 * qw;
                const float4 *m8 = reinterpret_cast<const float4 *>(msm + 8 * TS + r * TX) + 8 * qw;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 q = m4[j];
                    Mk[2 * j] = make_float2(q.x, q.y), Mk[2 * j + 1] = make_float2(q.z, q.w);
                }
                const float4 q8 = m8[tl];
                Mk8[0] = make_float2(q8.x, q8.y), Mk8[1] = make_float2(q8.z, q8.w);
            }
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(m_done);

            for (int g = 0; g < ngroups; ++g) {
                split_wait(&full[s], ph, abort_flag, p.status, 2);
                const float4 *ain0 = reinterpret_cast<const float4 *>(ring + s * STAGE + r * TX) + 8 * qw;  // in[g * CB], this row, this quarter
                float tot[CB];
#pragma unroll
                for (int cp = 0; cp < CB; cp += kSplitKU) {
                    const float4 *ain = ain0 + cp * (CHAN / 4);
                    float2 acc[kSplitKU][2], acc8[kSplitKU];
#pragma unroll
                    for (int u = 0; u < kSplitKU; ++u) {
                        const float4 a8 = ain[u * (CHAN / 4) + tl];
                        acc[u][0] = make_float2(0.f, 0.f), acc[u][1] = make_float2(0.f, 0.f);
                        acc8[u] = __ffma2_rn(make_float2(a8.x, a8.y), Mk8[0], make_float2(0.f, 0.f));
                        acc8[u] = __ffma2_rn(make_float2(a8.z, a8.w), Mk8[1], acc8[u]);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 av[kSplitKU];
#pragma unroll
                        for (int u = 0; u < kSplitKU; ++u) av[u] = ain[u * (CHAN / 4) + j];  // one 16-byte piece per quarter-warp
#pragma unroll
                        for (int u = 0; u < kSplitKU; ++u) {
                            acc[u][0] = __ffma2_rn(make_float2(av[u].x, av[u].y), Mk[2 * j], acc[u][0]);
                            acc[u][1] = __ffma2_rn(make_float2(av[u].z, av[u].w), Mk[2 * j + 1], acc[u][1]);
                        }
                    }
#pragma unroll
                    for (int u = 0; u < kSplitKU; ++u) {
                        const float sa = (acc[u][0].x + acc[u][0].y) + (acc[u][1].x + acc[u][1].y), sb = acc8[u].x + acc8[u].y;
                        // lanes 0-15 end up with tap tl summed over the quarter-warps, lanes 16-31 with tap 8
                        float v = (hi ? sb : sa) + __shfl_xor_sync(0xffffffffu, hi ? sa : sb, 16);
                        v += __shfl_xor_sync(0xffffffffu, v, 8);
                        float w8 = v;  // tap 8 also sums over the eight tap lanes (meaningful in lanes 16-31)
                        w8 += __shfl_xor_sync(0xffffffffu, w8, 1);
                        w8 += __shfl_xor_sync(0xffffffffu, w8, 2);
                        w8 += __shfl_xor_sync(0xffffffffu, w8, 4);
                        tot[cp + u] = hi ? w8 : v;
                    }
                }
                __syncwarp();
                if (lane == 0) tma::mbar_arrive(&empty[s]);
                if (tfinal < TAPS) {
#pragma unroll
                    for (int cc = 0; cc < CB; ++cc)
                        if (g * CB + cc < p.C) wslot[(g * CB + cc) * WPAD] += tot[cc];
                }
                if (++s == (uint32_t)S) s = 0, ph ^= 1u;
            }
        }
        }
    } else {
        // ===================================== X warps =====================================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSplitRegsX));
        const int r = warp, xq = lane;
        float bsum = 0.f;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tcount) {
            const int tx_i = (int)(tile % p.tiles_x);
            const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
            const long long nz = tile / tiles_per_plane;
            const int z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
            const int x0 = tx_i * TX, y0 = ty_i * TR;
            split_wait(table_full, tcount & 1u, abort_flag, p.status, 8);

            // XR rows per warp (r, r + 4, ...), each with four voxels per lane
            float2 M[XR][TAPS][2];  // pairs of neighbouring voxels
            bool valid[XR];
#pragma unroll
            for (int xr = 0; xr < XR; ++xr) {
                valid[xr] = (y0 + r + 4 * xr) < p.Y;
#pragma unroll
                for (int t = 0; t < TAPS; ++t) {
                    const float4 q = *reinterpret_cast<const float4 *>(msm + t * TS + (r + 4 * xr) * TX + 4 * xq);
                    M[xr][t][0] = make_float2(q.x, q.y), M[xr][t][1] = make_float2(q.z, q.w);
                }
                if (valid[xr]) bsum += (M[xr][TAPS / 2][0].x + M[xr][TAPS / 2][0].y) + (M[xr][TAPS / 2][1].x + M[xr][TAPS / 2][1].y);  // centre tap = m itself
            }
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(m_done);

            float *gi_row = p.gin + n * p.gi_sn + z * p.gi_sz + (int64_t)(y0 + r) * p.gi_sy + x0 + 4 * xq;
            for (int g = 0; g < ngroups; ++g) {
                split_wait(&full[s], ph, abort_flag, p.status, 2);
                const float *stage = ring + s * STAGE + r * TX + 4 * xq;
                const bool live = !*abort_flag;
                // two channels at a time: 8 XR independent FMA chains that share the M operands.
                // When C is odd the last pair's second channel reads a zero-filled stage and
                // whatever follows the weights in shared memory; its result is not stored.
#pragma unroll
                for (int cp = 0; cp < CB; cp += 2) {
                    const int c = g * CB + cp;
                    if (c < p.C) {
                        const float4 *wp0 = reinterpret_cast<const float4 *>(wsm + c * WPAD);
                        const float4 *wp1 = wp0 + WPAD / 4;
                        float gv0[XR][4], gv1[XR][4];
#pragma unroll
                        for (int xr = 0; xr < XR; ++xr) {
                            const float4 gq0 = ld4(stage + (CB + cp) * CHAN + 4 * xr * TX), gq1 = ld4(stage + (CB + cp + 1) * CHAN + 4 * xr * TX);
                            gv0[xr][0] = gq0.x, gv0[xr][1] = gq0.y, gv0[xr][2] = gq0.z, gv0[xr][3] = gq0.w;
                            gv1[xr][0] = gq1.x, gv1[xr][1] = gq1.y, gv1[xr][2] = gq1.z, gv1[xr][3] = gq1.w;
                        }
                        float4 wa = wp0[0], wb = wp1[0];
#pragma unroll
                        for (int i = 0; i < WPAD / 4; ++i) {
                            const float w0[4] = {wa.x, wa.y, wa.z, wa.w}, w1[4] = {wb.x, wb.y, wb.z, wb.w};
                            if (i + 1 < WPAD / 4) wa = wp0[i + 1], wb = wp1[i + 1];  // the next four taps, ahead of this quad's FMAs
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int t = 4 * i + q;
                                if (t < TAPS) {
#pragma unroll
                                    for (int xr = 0; xr < XR; ++xr) {
                                        gv0[xr][0] = fmaf(w0[q], M[xr][t][0].x, gv0[xr][0]), gv1[xr][0] = fmaf(w1[q], M[xr][t][0].x, gv1[xr][0]);
                                        gv0[xr][1] = fmaf(w0[q], M[xr][t][0].y, gv0[xr][1]), gv1[xr][1] = fmaf(w1[q], M[xr][t][0].y, gv1[xr][1]);
                                        gv0[xr][2] = fmaf(w0[q], M[xr][t][1].x, gv0[xr][2]), gv1[xr][2] = fmaf(w1[q], M[xr][t][1].x, gv1[xr][2]);
                                        gv0[xr][3] = fmaf(w0[q], M[xr][t][1].y, gv0[xr][3]), gv1[xr][3] = fmaf(w1[q], M[xr][t][1].y, gv1[xr][3]);
                                    }
                                }
                            }
                        }
#pragma unroll
                        for (int xr = 0; xr < XR; ++xr) {
                            // a channel that is the output of the layer below: hand its gradient over
                            // already multiplied by that layer's ReLU gate
                            if (c == p.mask_channel) {
                                const float4 a = ld4(stage + cp * CHAN + 4 * xr * TX);
                                gv0[xr][0] = a.x > 0.f ? gv0[xr][0] : 0.f;
                                gv0[xr][1] = a.y > 0.f ? gv0[xr][1] : 0.f;
                                gv0[xr][2] = a.z > 0.f ? gv0[xr][2] : 0.f;
                                gv0[xr][3] = a.w > 0.f ? gv0[xr][3] : 0.f;
                            }
                            if (c + 1 == p.mask_channel) {
                                const float4 a = ld4(stage + (cp + 1) * CHAN + 4 * xr * TX);
                                gv1[xr][0] = a.x > 0.f ? gv1[xr][0] : 0.f;
                                gv1[xr][1] = a.y > 0.f ? gv1[xr][1] : 0.f;
                                gv1[xr][2] = a.z > 0.f ? gv1[xr][2] : 0.f;
                                gv1[xr][3] = a.w > 0.f ? gv1[xr][3] : 0.f;
                            }
                            if (live && valid[xr]) {
                                float *dst = gi_row + (int64_t)(4 * xr) * p.gi_sy;
                                *reinterpret_cast<float4 *>(dst + c * p.gi_sc) = make_float4(gv0[xr][0], gv0[xr][1], gv0[xr][2], gv0[xr][3]);
                                if (c + 1 < p.C) *reinterpret_cast<float4 *>(dst + (c + 1) * p.gi_sc) = make_float4(gv1[xr][0], gv1[xr][1], gv1[xr][2], gv1[xr][3]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) tma::mbar_arrive(&empty[s]);
                if (++s == (uint32_t)S) s = 0, ph ^= 1u;
            }
        }
        if (p.part_b) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) bsum += __shfl_down_sync(0xffffffffu, bsum, off);
            if (lane == 0) red[r] = bsum;
        }
    }

    // ---- block epilogue: fixed-order sums of the K warps' slots, one partial per block ----
    tma::named_barrier(1, kSplitConsumers);
    if (!*abort_flag) {
        float *dst = p.part_k + (int64_t)blockIdx.x * p.C * TAPS;
        for (int i = tid; i < p.C * TAPS; i += kSplitConsumers) {
            const int c = i / TAPS, t = i - c * TAPS;
            float s_ = 0.f;
#pragma unroll
            for (int w = 0; w < kSplitKWarps; ++w) s_ += wacc[((size_t)w * p.C + c) * WPAD + t];
            dst[i] = s_;
        }
        if (p.part_b && tid == 0) {
            float s_ = 0.f;
#pragma unroll
            for (int w = 0; w < kSplitXWarps; ++w) s_ += red[w];
            p.part_b[blockIdx.x] = s_;
        }
    }
}

}  // namespace fast
}  // namespace msd

// Fused backward of one 3D MSD layer (one output channel, float32) with the INPUT gradient on
// the 5th-generation tensor cores (tcgen05, accumulator in tensor memory) and the WEIGHT
// gradient on the CUDA cores.  Same mathematics and buffers as fused_backward_kernel
// (fast_backward.cuh):
//     gin[c][q] += sum_t k[c][t] * M_t[q]           gk[c][t] += sum_q in[c][q] * M_t[q]
//
// Why this split.  A tcgen05.mma costs ~160 clocks whatever its shape (measured: M 64..128,
// N 16..256, K = 8 TF32), so only wide products pay.  The input gradient of a tile of 256
// voxels is  D[C x 256] = W[C x 32 taps] * T^T[32 x 256]:  N = 256, twelve instructions per
// tile whatever C is (4 steps of 8 taps x 3 products of the error-compensated split below) -
// 7.5 clocks per voxel against 27 FMAs per voxel AND CHANNEL on the CUDA cores.  The weight
// gradient contracts over the voxels, 8 per instruction, into a skinny C x 27 result: on the
// tensor cores it would need 40 clocks per voxel, more than the CUDA cores take for any C
// below ~70 (a kernel that does so was built and measured: 3.5 x slower than this one's
// predecessor).  So the weight gradient keeps the "K warps" of fast_backward_split.cuh,
// and the warps that used to compute the input gradient with 27 x 4 FMAs per lane and channel
// are gone.
//
// TF32 keeps 10 mantissa bits.  Both operands are split x = hi + lo (hi = x with its low 13
// bits cleared, lo = x - hi) and the product is formed as hi*hi' + lo*hi' + hi*lo' with float32
// accumulation ("3xTF32"): the result is as accurate as a float32 FMA chain.
//
// Per tile of 2 rows x 128 columns (256 voxels):
//   builders (4 warps)  halo rows of the gated gradient channel (TMA) -> rows of m -> the table
//                       M_t(voxel) twice: plain float32 [tap][voxel] for the K warps, and
//                       [voxel][tap] as hi / lo with the 128-byte swizzle (B operand of the MMA)
//   MMA issuer          12 x tcgen05.mma (M = 64 or 128 channels, N = 256) -> D in tensor memory
//   epilogue (4 warps)  thread = channel: D + gin -> gin, 64 bytes per thread and step, gin read
//                       from L2 (the producer prefetches the tile's gin with a bulk L2 prefetch)
//   K warps (16)        like those of the role-split kernel, but with half the voxels each so that
//                       twice as many fit: lane = (quarter-warp, tap lane), 4 taps x 8 voxels of M in
//                       registers (32 of its 80), activations streamed through a TMA ring of 8-channel
//                       stages; the two K warps of a 32-voxel unit take alternate stages
//   producers (2 warps) TMA: activations ring | halo rows of the next tile, L2 prefetch of gin
// The accumulator is double-buffered (2 x 256 of the 512 columns), so the MMA of the next tile
// overlaps this tile's epilogue.  Every hand-over is an mbarrier with a time-bounded wait.
//
// Requirements (checked by the host): X a multiple of 128, dilation <= 12, both gradients
// wanted, the gradient channel already gated, at most 128 input channels.
#pragma once
#include "fast_backward_split.cuh"
#include "umma.cuh"

namespace msd {
namespace fast {

constexpr int kHybTX = 128, kHybRows = 2, kHybNV = kHybTX * kHybRows;  // tile: 256 voxels = N of the MMA
constexpr int kHybCB = 8;                                              // channels per ring stage
constexpr int kHybThreads = 896;                                       // seven warpgroups
constexpr int kHybKUnits = 8;                                          // units of 32 voxels per tile; two K warps (alternate stages) each
constexpr int kHybEpilogueWarps = 4, kHybKWarp0 = 4, kHybKWarps = 2 * kHybKUnits, kHybProducerWarp = 20, kHybIssuerWarp = 21, kHybHaloWarp = 22,
              kHybBuilderWarp0 = 24;
constexpr int kHybBuilders = 128;
constexpr int kHybMaxStages = 8;
// Registers per thread after setmaxnreg.  The pool that setmaxnreg re-divides is what the block got
// at launch: 896 threads x 72 registers (the launch bound's 73, rounded down to a multiple of 8) =
// 64512 = 128 x (96 epilogue + 4 x 80 K warpgroups + 24 producers + 64 builders).  A sum above the
// pool would make setmaxnreg.inc wait forever; the launcher checks the compiled kernel against it.
constexpr int kHybRegsEpilogue = 96, kHybRegsK = 80, kHybRegsProducer = 24, kHybRegsBuilder = 64;
constexpr int kHybRegBudget = 128 * (kHybRegsEpilogue + (kHybKWarps / 4) * kHybRegsK + kHybRegsProducer + kHybRegsBuilder);
static_assert(kHybRegBudget <= kHybThreads * 72, "setmaxnreg budget exceeds the register pool");
constexpr int kHybHeaderBytes = 1024;
constexpr int kHybT1Bytes = kHybNV * 128;       // one copy (hi or lo) of T1[voxel][32 taps]
constexpr int kHybTS = kHybNV + 4;              // tap stride of the plain table (4 banks apart)
constexpr int kHybWaccPad = 28;

struct HybLayout {
    int mrows, w_bytes, hslot, halo_bytes, msm_bytes, stage_bytes, wacc_bytes;
    size_t total;
};
__host__ __device__ inline HybLayout hyb_layout(int C, int Dp, int stages) {
    HybLayout L;
    L.mrows = C <= 64 ? 64 : 128;
    L.w_bytes = 2 * L.mrows * 128;  // hi rows, then lo rows
    L.hslot = (kHybRows * (kHybTX + 2 * Dp) + 31) & ~31;
    L.halo_bytes = 9 * L.hslot * 4;
    L.msm_bytes = ((27 * kHybTS * 4) + 127) & ~127;
    L.stage_bytes = kHybCB * kHybNV * 4;
    L.wacc_bytes = kHybKUnits * C * kHybWaccPad * 4;  // one slot array per unit: its two K warps update disjoint channels
    L.total = (size_t)kHybHeaderBytes + 2 * kHybT1Bytes + L.w_bytes + L.halo_bytes + L.msm_bytes + (size_t)stages * L.stage_bytes + L.wacc_bytes;
    return L;
}

__device__ __forceinline__ void prefetch_l2_5d(const CUtensorMap *map, int c0, int c1, int c2, int c3, int c4) {
    asm volatile("cp.async.bulk.prefetch.tensor.5d.L2.global.tile [%0, {%1, %2, %3, %4, %5}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
                 : "memory");
}

__global__ void __launch_bounds__(kHybThreads, 1)
fused_backward3d_hybrid_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_gin_prefetch,
                               const __grid_constant__ CUtensorMap map_gout, const BwdParams p) {
    constexpr int RT = 9, TAPS = 27, TX = kHybTX, TR = kHybRows, NV = kHybNV, CB = kHybCB, KH = 32, TS = kHybTS;
    constexpr int CHAN = NV;          // floats of one channel in a ring stage
    constexpr int STAGE = CB * CHAN;  // floats of a ring stage
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw);  // [kHybMaxStages]
    uint64_t *empty = full + kHybMaxStages;
    uint64_t *halo_full = empty + kHybMaxStages;
    uint64_t *halo_empty = halo_full + 1;
    uint64_t *table_full = halo_empty + 1;  // the tables of a tile are complete
    uint64_t *m_done = table_full + 1;      // every K warp has its registers of M
    uint64_t *t1_free = m_done + 1;         // the MMAs that read T1 have completed
    uint64_t *d_full = t1_free + 1;         // [2] accumulator of a tile complete
    uint64_t *d_empty = d_full + 2;         // [2] ... read by the epilogue
    volatile int *abort_flag = reinterpret_cast<volatile int *>(d_empty + 2);
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(const_cast<int *>(abort_flag) + 1);
    float *red = reinterpret_cast<float *>(smem_raw + 512);

    const int S = p.stages, C = p.C;
    const HybLayout L = hyb_layout(C, p.Dp, S);
    const int TXP = TX + 2 * p.Dp, HSLOT = L.hslot;
    unsigned char *t1 = smem_raw + kHybHeaderBytes;  // hi copy, then lo copy
    unsigned char *wbuf = t1 + 2 * kHybT1Bytes;      // W hi rows, then lo rows
    float *rows = reinterpret_cast<float *>(wbuf + L.w_bytes);
    float *msm = rows + RT * HSLOT;
    float *ring = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(msm) + L.msm_bytes);
    float *wacc = ring + (size_t)S * STAGE;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((tma::smem_u32(smem_raw) & 1023u) != 0) {
        // the swizzled operands need 1024-byte aligned atoms; report instead of computing nonsense
        if (tid == 0) atomicCAS(p.status, 0, 21);
        return;
    }
    const int ngroups = (C + CB - 1) / CB;
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            tma::mbar_init(&full[s], 1);
            tma::mbar_init(&empty[s], kHybKUnits);  // the K warps of one parity
        }
        tma::mbar_init(halo_full, 1);
        tma::mbar_init(halo_empty, 1);
        tma::mbar_init(table_full, 1);
        tma::mbar_init(m_done, kHybKWarps);
        tma::mbar_init(t1_free, 1);
        for (int i = 0; i < 2; ++i) {
            tma::mbar_init(&d_full[i], 1);
            tma::mbar_init(&d_empty[i], kHybEpilogueWarps);
        }
        *abort_flag = 0;
        tma::fence_barrier_init();
    }
    // T1: the padding taps 27..31 of every voxel row stay zero for the whole kernel
    for (int i = tid; i < 2 * kHybT1Bytes / 16; i += kHybThreads) reinterpret_cast<float4 *>(t1)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    // W[c][t] as hi / lo, 128-byte swizzled rows of 32 taps (27 real); rows past C are zero
    for (int i = tid; i < L.mrows * 32; i += kHybThreads) {
        const int c = i >> 5, t = i & 31;
        const float w = (c < C && t < TAPS) ? p.k[c * TAPS + t] : 0.f;
        const float hi = umma::tf32_hi(w);
        const uint32_t off = umma::sw128_offset(c, t);
        *reinterpret_cast<float *>(wbuf + off) = hi;
        *reinterpret_cast<float *>(wbuf + L.mrows * 128 + off) = w - hi;
    }
    for (int i = tid; i < kHybKUnits * C * kHybWaccPad; i += kHybThreads) wacc[i] = 0.f;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) umma::tmem_alloc(tmem_base_slot, 512);
    tma::allow_dependents();
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    tma::grid_dependency_wait();
    const uint32_t tmem = *tmem_base_slot;

    const long long tiles_per_plane = (long long)p.tiles_x * p.tiles_y;
    auto tile_coords = [&](long long tile, int &n, int &z, int &y0, int &x0) {
        const int tx_i = (int)(tile % p.tiles_x);
        const int ty_i = (int)((tile / p.tiles_x) % p.tiles_y);
        const long long nz = tile / tiles_per_plane;
        z = p.z0 + (int)(nz % p.ZW), n = (int)(nz / p.ZW);
        x0 = tx_i * TX, y0 = ty_i * TR;
    };

    if (warp >= kHybProducerWarp && warp < kHybBuilderWarp0) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHybRegsProducer));
    if (warp == kHybProducerWarp) {
        // ------------------------- TMA producer of the activations -------------------------
        if (lane == 0) {
            tma::prefetch_tensormap(&map_in);
            uint32_t it = 0, s = 0, ph = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                int n, z, y0, x0;
                tile_coords(tile, n, z, y0, x0);
                for (int g = 0; g < ngroups; ++g, ++it) {
                    if (it >= (uint32_t)S) split_wait(&empty[s], ph ^ 1u, abort_flag, p.status, 1);
                    tma::mbar_arrive_expect_tx(&full[s], (uint32_t)(STAGE * 4));
                    // channels past C are outside the tensor map: zero-filled, no traffic
                    tma::tensor_g2s_5d(ring + (size_t)s * STAGE, &map_in, x0, y0, z, g * CB, n, &full[s]);
                    if (++s == (uint32_t)S) s = 0, ph ^= 1u;
                }
            }
        }
    } else if (warp == kHybHaloWarp) {
        // ------------- TMA producer of the halo rows; L2 prefetch of the gradients -------------
        if (lane == 0) {
            tma::prefetch_tensormap(&map_gout);
            tma::prefetch_tensormap(&map_gin_prefetch);
            const uint32_t halo_bytes = (uint32_t)(RT * TR * TXP * 4);
            auto prefetch_gin = [&](long long tile) {  // the whole tile of every channel, into L2, for the epilogue
                int n, z, y0, x0;
                tile_coords(tile, n, z, y0, x0);
                for (int c0 = 0; c0 < C; c0 += 64) prefetch_l2_5d(&map_gin_prefetch, x0, y0, z, c0, n);
            };
            if ((long long)blockIdx.x < p.num_tiles) prefetch_gin(blockIdx.x);
            uint32_t tc = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tc) {
                int n, z, y0, x0;
                tile_coords(tile, n, z, y0, x0);
                if (tc) split_wait(halo_empty, (tc - 1) & 1u, abort_flag, p.status, 5);  // the builders are done with the previous rows
                tma::mbar_arrive_expect_tx(halo_full, halo_bytes);
#pragma unroll 1
                for (int rt = 0; rt < RT; ++rt)
                    tma::tensor_g2s_5d(rows + rt * HSLOT, &map_gout, x0 - p.Dp, y0 + p.d * (1 - rt % 3), z + p.d * (1 - rt / 3), 0, n, halo_full);
                if (tile + gridDim.x < p.num_tiles) prefetch_gin(tile + gridDim.x);
            }
        }
    } else if (warp == kHybIssuerWarp) {
        // ------------------------------------ MMA issuer ------------------------------------
        if (lane == 0) {
            const uint32_t idesc = umma::idesc_tf32(L.mrows, NV, false, false);
            const uint32_t w_hi = tma::smem_u32(wbuf), w_lo = w_hi + L.mrows * 128;
            const uint32_t t_hi = tma::smem_u32(t1), t_lo = t_hi + kHybT1Bytes;
            uint32_t tc = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tc) {
                const int buf = tc & 1;
                split_wait(table_full, tc & 1u, abort_flag, p.status, 13);
                if (tc >= 2) split_wait(&d_empty[buf], ((tc >> 1) & 1u) ^ 1u, abort_flag, p.status, 14);
                umma::fence_after_sync();
                const uint32_t d = tmem + buf * NV;
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                    const uint64_t a_hi = umma::smem_desc_sw128(w_hi + 32 * ks, 0, 1024), a_lo = umma::smem_desc_sw128(w_lo + 32 * ks, 0, 1024);
                    const uint64_t b_hi = umma::smem_desc_sw128(t_hi + 32 * ks, 0, 1024), b_lo = umma::smem_desc_sw128(t_lo + 32 * ks, 0, 1024);
                    umma::mma_tf32(d, a_hi, b_hi, idesc, ks > 0);
                    umma::mma_tf32(d, a_lo, b_hi, idesc, 1);
                    umma::mma_tf32(d, a_hi, b_lo, idesc, 1);
                }
                umma::commit(&d_full[buf]);
                umma::commit(t1_free);
            }
        }
    } else if (warp >= kHybBuilderWarp0) {
        // ---------------- builders: the tables of the NEXT tile while the K warps stream ----------------
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHybRegsBuilder));
        const int btid = tid - kHybBuilderWarp0 * 32, bw = btid >> 5;
        uint32_t tc = 0;
        float bsum = 0.f;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tc) {
            int n, z, y0, x0;
            tile_coords(tile, n, z, y0, x0);
            split_wait(halo_full, tc & 1u, abort_flag, p.status, 6);
            split_fill_rows<kHybBuilders, kHybRows>(p, rows, nullptr, HSLOT, TXP, false, btid, n, z, y0, x0);
            if (tc) {
                split_wait(m_done, (tc - 1) & 1u, abort_flag, p.status, 7);    // the plain table has been read
                split_wait(t1_free, (tc - 1) & 1u, abort_flag, p.status, 18);  // ... and the MMAs are done with T1
            }
            tma::named_barrier(3, kHybBuilders);
            const bool fold_l = x0 == 0, fold_r = x0 + TX == p.X;
            // thread = voxel (two per thread): its 27 values of M from the nine rows, then one row of
            // T1 as 128-bit stores (hi and lo) and 27 plain stores for the K warps
#pragma unroll 1
            for (int vv = 0; vv < NV / kHybBuilders; ++vv) {
                const int vox = btid + kHybBuilders * vv, r = vox / TX, ci = vox % TX;
                float m[28];
#pragma unroll
                for (int rt = 0; rt < RT; ++rt) {
                    const float *row = rows + rt * HSLOT + r * TXP + p.Dp;  // row[i] <-> image x = x0 + i
                    float v0 = row[ci + p.d], v1 = row[ci], v2 = row[ci - p.d];
                    if (fold_l && ci < p.d) v0 += row[p.d - 1 - ci];
                    if (fold_r && ci >= TX - p.d) v2 += row[2 * TX - 1 - p.d - ci];
                    m[3 * rt] = v0, m[3 * rt + 1] = v1, m[3 * rt + 2] = v2;
                }
                m[27] = 0.f;
                bsum += m[13];
#pragma unroll
                for (int t = 0; t < TAPS; ++t) msm[t * TS + vox] = m[t];
                unsigned char *row1 = t1 + vox * 128;
#pragma unroll
                for (int q = 0; q < 7; ++q) {
                    float4 h4, l4;
                    h4.x = umma::tf32_hi(m[4 * q]), h4.y = umma::tf32_hi(m[4 * q + 1]), h4.z = umma::tf32_hi(m[4 * q + 2]), h4.w = umma::tf32_hi(m[4 * q + 3]);
                    l4.x = m[4 * q] - h4.x, l4.y = m[4 * q + 1] - h4.y, l4.z = m[4 * q + 2] - h4.z, l4.w = m[4 * q + 3] - h4.w;
                    const int off = (q ^ (vox & 7)) << 4;
                    *reinterpret_cast<float4 *>(row1 + off) = h4;
                    *reinterpret_cast<float4 *>(row1 + kHybT1Bytes + off) = l4;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // T1 is read by the tensor cores, the rows are rewritten by TMA
            tma::named_barrier(3, kHybBuilders);
            if (btid == 0) {
                tma::mbar_arrive(halo_empty);
                tma::mbar_arrive(table_full);
            }
        }
        if (p.part_b) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) bsum += __shfl_down_sync(0xffffffffu, bsum, off);
            if (lane == 0) red[bw] = bsum;
            tma::named_barrier(3, kHybBuilders);
            if (btid == 0 && !*abort_flag) p.part_b[blockIdx.x] = (red[0] + red[1]) + (red[2] + red[3]);
        }
    } else if (warp >= kHybKWarp0 && warp < kHybKWarp0 + kHybKWarps) {
        // ===================================== K warps =====================================
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kHybRegsK));
        // unit = 32 voxels of the tile (row r, columns 32 xs ..); the warps of parity 0 / 1 take the even /
        // odd ring stages.  lane = (qw, tl): taps tl + 8 {0..3}; voxels 4 (4 j + qw) + {0..3}, j = 0..1.
        const int kw = warp - kHybKWarp0, unit = kw & (kHybKUnits - 1), parity = kw / kHybKUnits, r = unit >> 2, xs = unit & 3;
        const int qw = lane >> 3, tl = lane & 7;
        const bool hi = (lane & 16) != 0, mid = (lane & 8) != 0;
        const int tfinal = tl + 8 * ((hi ? 2 : 0) + (mid ? 1 : 0));  // the tap whose sum this lane ends up with
        float *wslot = wacc + (size_t)unit * C * kHybWaccPad + tfinal;
        uint32_t tc = 0, s = 0, ph = 0;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tc) {
            split_wait(table_full, tc & 1u, abort_flag, p.status, 8);
            float2 Mk[4][KH / 8];
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const int ta = tl + 8 * a;
                const float4 *m4 = reinterpret_cast<const float4 *>(msm + (ta < TAPS ? ta : 0) * TS + r * TX + KH * xs);
#pragma unroll
                for (int j = 0; j < KH / 16; ++j) {
                    float4 q = m4[4 * j + qw];
                    if (ta >= TAPS) q = make_float4(0.f, 0.f, 0.f, 0.f);
                    Mk[a][2 * j] = make_float2(q.x, q.y), Mk[a][2 * j + 1] = make_float2(q.z, q.w);
                }
            }
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(m_done);
            for (int g = 0; g < ngroups; ++g) {
                if ((g & 1) == parity) {
                    split_wait(&full[s], ph, abort_flag, p.status, 2);
                    const float4 *ain0 = reinterpret_cast<const float4 *>(ring + (size_t)s * STAGE + r * TX + KH * xs) + qw;
                    float tot[CB];
#pragma unroll
                    for (int cp = 0; cp < CB; cp += 2) {
                        const float4 *ain = ain0 + cp * (CHAN / 4);
                        float4 av[2][KH / 16];
#pragma unroll
                        for (int u = 0; u < 2; ++u)
#pragma unroll
                            for (int j = 0; j < KH / 16; ++j) av[u][j] = ain[u * (CHAN / 4) + 4 * j];
                        float2 acc[2][4];
#pragma unroll
                        for (int u = 0; u < 2; ++u)
#pragma unroll
                            for (int a = 0; a < 4; ++a) acc[u][a] = make_float2(0.f, 0.f);
#pragma unroll
                        for (int j = 0; j < KH / 16; ++j)
#pragma unroll
                            for (int a = 0; a < 4; ++a)
#pragma unroll
                                for (int u = 0; u < 2; ++u) {
                                    acc[u][a] = __ffma2_rn(make_float2(av[u][j].x, av[u][j].y), Mk[a][2 * j], acc[u][a]);
                                    acc[u][a] = __ffma2_rn(make_float2(av[u][j].z, av[u][j].w), Mk[a][2 * j + 1], acc[u][a]);
                                }
                        float k0[2], k1[2];
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const float s0 = acc[u][0].x + acc[u][0].y, s1 = acc[u][1].x + acc[u][1].y;
                            const float s2 = acc[u][2].x + acc[u][2].y, s3 = acc[u][3].x + acc[u][3].y;
                            k0[u] = (hi ? s2 : s0) + __shfl_xor_sync(0xffffffffu, hi ? s0 : s2, 16);
                            k1[u] = (hi ? s3 : s1) + __shfl_xor_sync(0xffffffffu, hi ? s1 : s3, 16);
                        }
#pragma unroll
                        for (int u = 0; u < 2; ++u) tot[cp + u] = (mid ? k1[u] : k0[u]) + __shfl_xor_sync(0xffffffffu, mid ? k0[u] : k1[u], 8);
                    }
                    __syncwarp();
                    if (lane == 0) tma::mbar_arrive(&empty[s]);
                    if (tfinal < TAPS) {
#pragma unroll
                        for (int cc = 0; cc < CB; ++cc)
                            if (g * CB + cc < C) wslot[(g * CB + cc) * kHybWaccPad] += tot[cc];
                    }
                }
                if (++s == (uint32_t)S) s = 0, ph ^= 1u;
            }
        }
    } else if (warp < kHybEpilogueWarps) {
        // ------------------------------------ epilogue warps ------------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kHybRegsEpilogue));
        // thread = channel.  M = 64: channel c sits in lane 32 (c / 16) + (c % 16) of the accumulator
        // (the upper half of each warp's lanes holds nothing); M = 128: in lane c.
        const int ch = L.mrows == 64 ? ((lane < 16) ? 16 * warp + lane : -1) : 32 * warp + lane;
        const bool has_channel = ch >= 0 && ch < C;
        uint32_t tc = 0;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tc) {
            int n, z, y0, x0;
            tile_coords(tile, n, z, y0, x0);
            const int buf = tc & 1;
            const int cc = has_channel ? ch : 0;
            float *gbase = p.gin + n * p.gi_sn + (int64_t)cc * p.gi_sc + z * p.gi_sz + (int64_t)y0 * p.gi_sy + x0;
            const float *ibase = p.in + n * p.in_sn + (int64_t)cc * p.in_sc + z * p.in_sz + (int64_t)y0 * p.in_sy + x0;
            const bool gate_here = has_channel && ch == p.mask_channel;
            // 16 steps of 16 voxels; the gradients of three steps are in flight ahead of the sums
            constexpr int STEPS = NV / 16, AHEAD = 2;
            float4 g[AHEAD][4];
            auto row_ok = [&](int q) { return has_channel && (y0 + (q * 16) / TX) < p.Y; };
            auto goff = [&](int q) { return (int64_t)((q * 16) / TX) * p.gi_sy + (q * 16) % TX; };
            auto load = [&](int q, float4 (&dst)[4]) {
                if (row_ok(q)) {
                    const float4 *src = reinterpret_cast<const float4 *>(gbase + goff(q));
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[i] = src[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            };
#pragma unroll
            for (int q = 0; q < AHEAD; ++q) load(q, g[q]);
            split_wait(&d_full[buf], (tc >> 1) & 1u, abort_flag, p.status, 19);
            umma::fence_after_sync();
            const bool live = !*abort_flag;
            const uint32_t d = tmem + buf * NV + ((uint32_t)(32 * warp) << 16);
            uint32_t acc[2][16];  // the sums of a step arrive while the previous step is added and stored
            umma::tmem_ld16_issue(d, acc[0]);
#pragma unroll
            for (int q = 0; q < STEPS; ++q) {
                umma::tmem_ld_wait();
                if (q + 1 < STEPS) umma::tmem_ld16_issue(d + 16 * (q + 1), acc[(q + 1) & 1]);
                const uint32_t(&a)[16] = acc[q & 1];
                float4(&cur)[4] = g[q % AHEAD];
                float4 out[4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    out[i] = make_float4(cur[i].x + __uint_as_float(a[4 * i]), cur[i].y + __uint_as_float(a[4 * i + 1]),
                                         cur[i].z + __uint_as_float(a[4 * i + 2]), cur[i].w + __uint_as_float(a[4 * i + 3]));
                if (gate_here && row_ok(q)) {
                    // this channel is the output of the layer below: hand its gradient over gated
                    const float4 *a4 = reinterpret_cast<const float4 *>(ibase + (int64_t)((q * 16) / TX) * p.in_sy + (q * 16) % TX);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 av = a4[i];
                        out[i].x = av.x > 0.f ? out[i].x : 0.f, out[i].y = av.y > 0.f ? out[i].y : 0.f;
                        out[i].z = av.z > 0.f ? out[i].z : 0.f, out[i].w = av.w > 0.f ? out[i].w : 0.f;
                    }
                }
                if (live && row_ok(q)) {
                    float4 *dst = reinterpret_cast<float4 *>(gbase + goff(q));
#pragma unroll
                    for (int i = 0; i < 4; ++i) dst[i] = out[i];
                }
                if (q + AHEAD < STEPS) load(q + AHEAD, g[q % AHEAD]);
            }
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&d_empty[buf]);
        }
    }

    // ---- block epilogue: fixed-order sums of the K warps' slots, one partial per block ----
    umma::fence_before_sync();
    __syncthreads();
    if (!*abort_flag) {
        float *dst = p.part_k + (int64_t)blockIdx.x * C * TAPS;
        for (int i = tid; i < C * TAPS; i += kHybThreads) {
            const int c = i / TAPS, t = i - c * TAPS;
            float s_ = 0.f;
#pragma unroll
            for (int w = 0; w < kHybKUnits; ++w) s_ += wacc[((size_t)w * C + c) * kHybWaccPad + t];
            dst[i] = s_;
        }
    }
    if (warp == 0) umma::tmem_dealloc(tmem, 512);
}

}  // namespace fast
}  // namespace msd

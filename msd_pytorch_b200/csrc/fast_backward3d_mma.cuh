// Fused backward of one 3D MSD layer (one output channel, float32) on the 5th-generation
// tensor cores (tcgen05, accumulators in tensor memory).  Same mathematics and buffers as
// fused_backward_kernel (fast_backward.cuh):
//     gin[c][q] += sum_t k[c][t] * M_t[q]           gk[c][t] += sum_q in[c][q] * M_t[q]
// With the table M_t[q] of the layer's single gated gradient channel in hand, both sums are
// dense contractions over that table.  Per stage of 64 voxels (half a tile row):
//     G1:  D1[64 voxels x C]    = T[64 x 32 taps]  * W^T[32 taps x C]      (input gradient)
//     G2:  D2[C x 32 taps]     += In[C x 64 voxels] * T^T[64 voxels x 32]   (weight gradient)
// Both run as kind::tf32 MMAs with float32 accumulation.  TF32 keeps 10 mantissa bits, so every
// operand is split x = hi + lo (hi = x with its low 13 bits cleared, lo = x - hi) and each
// product is computed as hi*hi' + lo*hi' + hi*lo' ("3xTF32"), which restores float32-level
// accuracy (the dropped lo*lo' term is ~2^-22 relative).  D2 stays in tensor memory for the
// whole kernel and is read once at the end; D1 is read per stage by the epilogue warps, which
// add it to gin straight from / to global memory (thread = voxel, so every access of a warp
// is one contiguous run).
//
// All operands are K-major with the 128-byte swizzle:
//   T1[voxel][tap]      A of G1 (hi and lo copies)            written by the builder warps
//   T2[tap][voxel]      B of G2 (rows 0-31 hi taps, 32-63 lo)  written by the builder warps
//   W[channel][tap]     B of G1 (hi and lo copies)            written once per block
//   In[channel][voxel]  A of G2: TMA boxes of 32 voxels x C channels (a tensor map whose second
//                       dimension is the channel), rewritten in place as hi and, beside it, lo
//                       by the splitter warps
// Rows of In beyond the layer's channels (the MMA reads 64 or 128 rows) hold whatever follows
// in shared memory; they only reach accumulator rows that are never read.
//
// Warps:  0-3 epilogue | 4 TMA producer of In and gin | 5 MMA issuer | 6 TMA producer of the halo rows
//         7-8 splitters | 9-12 builders.  Every hand-over is an mbarrier with a bounded wait.
//
// Requirements (checked by the host): X a multiple of 128, dilation <= 12, both gradients
// wanted, the gradient channel already gated, at most 128 input channels.
#pragma once
#include "fast_backward3d_split.cuh"
#include "umma.cuh"

namespace msd {
namespace fast {

constexpr int kMmaTX = 128;       // tile columns
constexpr int kMmaRows = 2;       // tile rows (granularity of the halo fetch)
constexpr int kMmaSV = 64;        // voxels per stage = M of G1
constexpr int kMmaStagesPerTile = kMmaRows * (kMmaTX / kMmaSV);
constexpr int kMmaThreads = 416;  // 13 warps
constexpr int kMmaEpilogueWarps = 4;
constexpr int kMmaInProducerWarp = 4, kMmaIssuerWarp = 5, kMmaHaloProducerWarp = 6;
constexpr int kMmaSplitWarp0 = 7, kMmaSplitters = 64;
constexpr int kMmaBuilderWarp0 = 9, kMmaBuilders = 128;
constexpr int kMmaMaxStages = 6;
constexpr int kMmaHeaderBytes = 1024;
constexpr int kMmaTableBytes = 32768;  // per slot: T1 hi 8 KB, T1 lo 8 KB, T2 16 KB
constexpr int kMmaTmemCols = 512;
constexpr int kMmaD2Col = 0, kMmaD1Col = 64;  // D2: 64 columns; D1: two buffers of up to 128 columns

struct MmaLayout {
    int C8, C16, in_stage_bytes, gin_stage_bytes, w_bytes, hslot, halo_bytes;
    size_t total;
};
__host__ __device__ inline MmaLayout mma_layout(int C, int Dp, int stages, int gin_stages) {
    MmaLayout L;
    L.C8 = (C + 7) & ~7;
    L.C16 = (C + 15) & ~15;
    L.in_stage_bytes = 2 * (kMmaSV / 32) * L.C8 * 128;  // hi chunks, then lo chunks
    L.gin_stage_bytes = L.C8 * kMmaSV * 4;              // [channel][64 voxels], dense
    L.w_bytes = 2 * L.C16 * 128;                        // hi rows, then lo rows
    L.hslot = (kMmaRows * (kMmaTX + 2 * Dp) + 31) & ~31;
    L.halo_bytes = 9 * L.hslot * 4;
    // header | In ring | tables (2 slots) | W | halo rows (2 buffers) | gin ring; 16 KB of slack after
    // the In ring is provided by the tables themselves (the MMA may read 128 rows from a chunk's base)
    L.total = (size_t)kMmaHeaderBytes + (size_t)stages * L.in_stage_bytes + 2 * kMmaTableBytes + ((L.w_bytes + 1023) & ~1023) +
              2 * (size_t)L.halo_bytes + (size_t)gin_stages * L.gin_stage_bytes;
    return L;
}

__global__ void __launch_bounds__(kMmaThreads, 1)
fused_backward3d_mma_kernel(const __grid_constant__ CUtensorMap map_in, const __grid_constant__ CUtensorMap map_gin,
                            const __grid_constant__ CUtensorMap map_gout, const BwdParams p) {
    constexpr int RT = 9, TAPS = 27, TX = kMmaTX, TR = kMmaRows, SV = kMmaSV, SPT = kMmaStagesPerTile;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    uint64_t *full_in = reinterpret_cast<uint64_t *>(smem_raw);  // [kMmaMaxStages]
    uint64_t *in_ready = full_in + kMmaMaxStages;
    uint64_t *empty_in = in_ready + kMmaMaxStages;
    uint64_t *halo_full = empty_in + kMmaMaxStages;  // [2]
    uint64_t *halo_empty = halo_full + 2;            // [2]
    uint64_t *table_full = halo_empty + 2;           // [2]
    uint64_t *table_empty = table_full + 2;          // [2]
    uint64_t *d1_full = table_empty + 2;             // [2]
    uint64_t *d1_empty = d1_full + 2;                // [2]
    uint64_t *gin_full = d1_empty + 2;               // [kMmaMaxStages]
    uint64_t *gin_empty = gin_full + kMmaMaxStages;  // [kMmaMaxStages]
    uint64_t *final_bar = gin_empty + kMmaMaxStages;
    volatile int *abort_flag = reinterpret_cast<volatile int *>(final_bar + 1);
    uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(const_cast<int *>(abort_flag) + 1);
    float *red = reinterpret_cast<float *>(smem_raw + 512);  // bias partials of the builder warps

    const int S = p.stages, SG = p.stages2;
    const MmaLayout L = mma_layout(p.C, p.Dp, S, SG);
    const int C = p.C, C8 = L.C8, C16 = L.C16;
    const int TXP = TX + 2 * p.Dp, HSLOT = L.hslot;
    unsigned char *in_ring = smem_raw + kMmaHeaderBytes;
    unsigned char *tables = in_ring + (size_t)S * L.in_stage_bytes;
    unsigned char *wbuf = tables + 2 * kMmaTableBytes;
    float *halo = reinterpret_cast<float *>(wbuf + ((L.w_bytes + 1023) & ~1023));
    unsigned char *gin_ring = reinterpret_cast<unsigned char *>(halo) + 2 * (size_t)L.halo_bytes;
    const int chunk_bytes = C8 * 128;               // one 32-voxel chunk of In: C8 rows of 128 bytes
    const int in_half = (SV / 32) * chunk_bytes;    // hi part of a stage; the lo part follows

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if ((tma::smem_u32(smem_raw) & 1023u) != 0) {
        // the swizzled operands need 1024-byte aligned atoms; report instead of computing nonsense
        if (tid == 0) atomicCAS(p.status, 0, 21);
        return;
    }
    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            tma::mbar_init(&full_in[s], 1);
            tma::mbar_init(&in_ready[s], 1);
            tma::mbar_init(&empty_in[s], 1);
        }
        for (int s = 0; s < SG; ++s) {
            tma::mbar_init(&gin_full[s], 1);
            tma::mbar_init(&gin_empty[s], kMmaEpilogueWarps);
        }
        for (int i = 0; i < 2; ++i) {
            tma::mbar_init(&halo_full[i], 1);
            tma::mbar_init(&halo_empty[i], 1);
            tma::mbar_init(&table_full[i], 1);
            tma::mbar_init(&table_empty[i], 1);
            tma::mbar_init(&d1_full[i], 1);
            tma::mbar_init(&d1_empty[i], kMmaEpilogueWarps);
        }
        tma::mbar_init(final_bar, 1);
        *abort_flag = 0;
        tma::fence_barrier_init();
    }
    // zero the In ring and the tables once: the padding rows / taps of the operands stay zero
    for (int i = tid; i < (int)(((size_t)S * L.in_stage_bytes + 2 * kMmaTableBytes) / 16); i += kMmaThreads)
        reinterpret_cast<float4 *>(in_ring)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    // W[c][t] as hi / lo, 128-byte swizzled rows of 32 taps (27 real), C16 rows each
    for (int i = tid; i < C16 * 32; i += kMmaThreads) {
        const int c = i >> 5, t = i & 31;
        const float w = (c < C && t < TAPS) ? p.k[c * TAPS + t] : 0.f;
        const float hi = umma::tf32_hi(w);
        const uint32_t off = umma::sw128_offset(c, t);
        *reinterpret_cast<float *>(wbuf + off) = hi;
        *reinterpret_cast<float *>(wbuf + C16 * 128 + off) = w - hi;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) umma::tmem_alloc(tmem_base_slot, kMmaTmemCols);
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

    if (warp == kMmaInProducerWarp) {
        // ------------------------- TMA producer of the activations -------------------------
        if (lane == 0) {
            tma::prefetch_tensormap(&map_in);
            tma::prefetch_tensormap(&map_gin);
            uint32_t it = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                int n, z, y0, x0;
                tile_coords(tile, n, z, y0, x0);
                for (int st = 0; st < SPT; ++st, ++it) {
                    const int s = it % S, r = st / (TX / SV), h = st % (TX / SV);
                    if (it >= (uint32_t)S) tma::wait_parity(&empty_in[s], ((it / S) & 1u) ^ 1u, abort_flag, p.status, 11);
                    tma::mbar_arrive_expect_tx(&full_in[s], (uint32_t)in_half);
                    unsigned char *dst = in_ring + (size_t)s * L.in_stage_bytes;
                    // coordinates (x, channel, y, z, n); channels past C are zero-filled
#pragma unroll
                    for (int j = 0; j < SV / 32; ++j) tma::tensor_g2s_5d(dst + j * chunk_bytes, &map_in, x0 + SV * h + 32 * j, 0, y0 + r, z, n, &full_in[s]);
                    // the same voxels of every channel of the gradients, for the epilogue
                    const int sg = it % SG;
                    if (it >= (uint32_t)SG) tma::wait_parity(&gin_empty[sg], ((it / SG) & 1u) ^ 1u, abort_flag, p.status, 22);
                    tma::mbar_arrive_expect_tx(&gin_full[sg], (uint32_t)L.gin_stage_bytes);
                    tma::tensor_g2s_5d(gin_ring + (size_t)sg * L.gin_stage_bytes, &map_gin, x0 + SV * h, y0 + r, z, 0, n, &gin_full[sg]);
                }
            }
        }
    } else if (warp == kMmaHaloProducerWarp) {
        // ---------------- TMA producer of the halo rows of the gradient channel ----------------
        if (lane == 0) {
            tma::prefetch_tensormap(&map_gout);
            const uint32_t halo_bytes = (uint32_t)(RT * TR * TXP * 4);
            uint32_t tc = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tc) {
                int n, z, y0, x0;
                tile_coords(tile, n, z, y0, x0);
                const int hb = tc & 1;
                if (tc >= 2) tma::wait_parity(&halo_empty[hb], ((tc >> 1) & 1u) ^ 1u, abort_flag, p.status, 12);
                tma::mbar_arrive_expect_tx(&halo_full[hb], halo_bytes);
                float *rows = halo + (size_t)hb * RT * HSLOT;
#pragma unroll 1
                for (int rt = 0; rt < RT; ++rt)
                    tma::tensor_g2s_5d(rows + rt * HSLOT, &map_gout, x0 - p.Dp, y0 + p.d * (1 - rt % 3), z + p.d * (1 - rt / 3), 0, n, &halo_full[hb]);
            }
        }
    } else if (warp == kMmaIssuerWarp) {
        // ------------------------------------ MMA issuer ------------------------------------
        if (lane == 0) {
            const int m2 = C <= 64 ? 64 : 128;  // rows of In the weight-gradient MMA reads
            const uint32_t idesc_g1 = umma::idesc_tf32(SV, C16, false, false);
            const uint32_t idesc_g2a = umma::idesc_tf32(m2, 64, false, false);
            const uint32_t idesc_g2b = umma::idesc_tf32(m2, 32, false, false);
            const uint32_t w_hi = tma::smem_u32(wbuf), w_lo = w_hi + C16 * 128;
            uint32_t it = 0;
            for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
                for (int st = 0; st < SPT; ++st, ++it) {
                    const int s = it % S, slot = it & 1, buf = it & 1;
                    const uint32_t tab = tma::smem_u32(tables + slot * kMmaTableBytes);
                    const uint32_t t1_hi = tab, t1_lo = tab + 8192, t2 = tab + 16384;
                    tma::wait_parity(&table_full[slot], (it >> 1) & 1u, abort_flag, p.status, 13);
                    if (it >= 2) tma::wait_parity(&d1_empty[buf], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, 14);
                    umma::fence_after_sync();
                    // G1: D1[buf] = T1 * W^T  (three products per 8 taps)
                    const uint32_t d1 = tmem + kMmaD1Col + buf * 128;
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t a_hi = umma::smem_desc_sw128(t1_hi + 32 * ks, 0, 1024), a_lo = umma::smem_desc_sw128(t1_lo + 32 * ks, 0, 1024);
                        const uint64_t b_hi = umma::smem_desc_sw128(w_hi + 32 * ks, 0, 1024), b_lo = umma::smem_desc_sw128(w_lo + 32 * ks, 0, 1024);
                        umma::mma_tf32(d1, a_hi, b_hi, idesc_g1, ks > 0);
                        umma::mma_tf32(d1, a_lo, b_hi, idesc_g1, 1);
                        umma::mma_tf32(d1, a_hi, b_lo, idesc_g1, 1);
                    }
                    umma::commit(&d1_full[buf]);
                    // G2: D2 += In * T2^T  (hi x [hi | lo] as one N = 64 product, lo x hi as N = 32)
                    tma::wait_parity(&in_ready[s], (it / S) & 1u, abort_flag, p.status, 15);
                    umma::fence_after_sync();
                    const uint32_t in_hi = tma::smem_u32(in_ring + (size_t)s * L.in_stage_bytes), in_lo = in_hi + in_half;
                    const uint32_t d2 = tmem + kMmaD2Col;
#pragma unroll
                    for (int j = 0; j < SV / 32; ++j)
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t b = umma::smem_desc_sw128(t2 + j * 8192 + 32 * ks, 0, 1024);
                            umma::mma_tf32(d2, umma::smem_desc_sw128(in_hi + j * chunk_bytes + 32 * ks, 0, 1024), b, idesc_g2a, (it | j | ks) != 0);
                            umma::mma_tf32(d2, umma::smem_desc_sw128(in_lo + j * chunk_bytes + 32 * ks, 0, 1024), b, idesc_g2b, 1);
                        }
                    umma::commit(&empty_in[s]);
                    umma::commit(&table_empty[slot]);
                }
            }
            umma::commit(final_bar);
        }
    } else if (warp >= kMmaSplitWarp0 && warp < kMmaBuilderWarp0) {
        // ------------- splitters: In -> hi (in place) and lo (beside it), per stage -------------
        const int stid = tid - kMmaSplitWarp0 * 32;
        uint32_t it = 0;
        const int units = in_half / 16;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
            for (int st = 0; st < SPT; ++st, ++it) {
                const int s = it % S;
                tma::wait_parity(&full_in[s], (it / S) & 1u, abort_flag, p.status, 16);
                float4 *hi = reinterpret_cast<float4 *>(in_ring + (size_t)s * L.in_stage_bytes);
                float4 *lo = reinterpret_cast<float4 *>(in_ring + (size_t)s * L.in_stage_bytes + in_half);
                for (int u = stid; u < units; u += kMmaSplitters) {
                    const float4 v = hi[u];
                    float4 h4, l4;
                    h4.x = umma::tf32_hi(v.x), h4.y = umma::tf32_hi(v.y), h4.z = umma::tf32_hi(v.z), h4.w = umma::tf32_hi(v.w);
                    l4.x = v.x - h4.x, l4.y = v.y - h4.y, l4.z = v.z - h4.z, l4.w = v.w - h4.w;
                    hi[u] = h4;
                    lo[u] = l4;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tma::named_barrier(2, kMmaSplitters);
                if (stid == 0) tma::mbar_arrive(&in_ready[s]);
            }
        }
    } else if (warp >= kMmaBuilderWarp0) {
        // ---------------- builders: halo rows -> rows of m -> the two tables, per stage ----------------
        const int btid = tid - kMmaBuilderWarp0 * 32, bw = btid >> 5;
        uint32_t it = 0, tc = 0;
        float bsum = 0.f;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++tc) {
            int n, z, y0, x0;
            tile_coords(tile, n, z, y0, x0);
            const int hb = tc & 1;
            float *rows = halo + (size_t)hb * RT * HSLOT;
            tma::wait_parity(&halo_full[hb], (tc >> 1) & 1u, abort_flag, p.status, 17);
            split_fill_rows<kMmaBuilders, kMmaRows>(p, rows, nullptr, HSLOT, TXP, false, btid, n, z, y0, x0);
            tma::named_barrier(3, kMmaBuilders);
            const bool fold_l = x0 == 0, fold_r = x0 + TX == p.X;
            for (int st = 0; st < SPT; ++st, ++it) {
                const int slot = it & 1, r = st / (TX / SV), h = st % (TX / SV);
                unsigned char *tab = tables + slot * kMmaTableBytes;
                if (it >= 2) tma::wait_parity(&table_empty[slot], ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, 18);
                // one tap per warp and step; lanes on consecutive voxels (two runs of 32)
#pragma unroll 1
                for (int t = bw; t < TAPS; t += kMmaBuilders / 32) {
                    const int rt = t / 3, tx = t - 3 * rt;
                    const float *row = rows + rt * HSLOT + r * TXP + p.Dp;  // row[i] <-> image x = x0 + i
#pragma unroll
                    for (int k = 0; k < SV / 32; ++k) {
                        const int ci = SV * h + 32 * k + lane;  // column inside the tile
                        float v = row[ci - p.d * (tx - 1)];
                        if (tx == 0 && fold_l && ci < p.d) v += row[p.d - 1 - ci];
                        if (tx == 2 && fold_r && ci >= TX - p.d) v += row[2 * TX - 1 - p.d - ci];
                        if (t == 13) bsum += v;
                        const float hi = umma::tf32_hi(v), lo = v - hi;
                        const int vox = 32 * k + lane;  // voxel inside the stage
                        const uint32_t o1 = umma::sw128_offset(vox, t);
                        *reinterpret_cast<float *>(tab + o1) = hi;
                        *reinterpret_cast<float *>(tab + 8192 + o1) = lo;
                        const uint32_t o2 = (uint32_t)(16384 + k * 8192) + umma::sw128_offset(t, lane);
                        *reinterpret_cast<float *>(tab + o2) = hi;
                        *reinterpret_cast<float *>(tab + o2 + 32 * 128) = lo;
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                tma::named_barrier(3, kMmaBuilders);
                if (btid == 0) tma::mbar_arrive(&table_full[slot]);
            }
            // the rows are no longer needed: the halo producer may overwrite this buffer
            if (btid == 0) tma::mbar_arrive(&halo_empty[hb]);
        }
        if (p.part_b) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) bsum += __shfl_down_sync(0xffffffffu, bsum, off);
            if (lane == 0) red[bw] = bsum;
            tma::named_barrier(3, kMmaBuilders);
            if (btid == 0 && !*abort_flag) p.part_b[blockIdx.x] = (red[0] + red[1]) + (red[2] + red[3]);
        }
    } else {
        // ------------------------------------ epilogue warps ------------------------------------
        // D1 (M = 64): voxel i of the stage sits in lane 32 (i / 16) + (i % 16); the upper half
        // of each warp's lanes holds nothing.
        const bool has_voxel = lane < 16;
        const int vox = 16 * warp + (lane & 15);
        uint32_t it = 0;
        for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
            int n, z, y0, x0;
            tile_coords(tile, n, z, y0, x0);
            for (int st = 0; st < SPT; ++st, ++it) {
                const int buf = it & 1, r = st / (TX / SV), h = st % (TX / SV);
                const bool valid = has_voxel && (y0 + r) < p.Y;
                const int64_t voff = (int64_t)(y0 + r) * p.gi_sy + x0 + SV * h + vox;
                float *gp = p.gin + n * p.gi_sn + z * p.gi_sz + voff;
                const float *ip = p.in + n * p.in_sn + z * p.in_sz + (int64_t)(y0 + r) * p.in_sy + x0 + SV * h + vox;
                const int sg = it % SG;
                const float *gs = reinterpret_cast<const float *>(gin_ring + (size_t)sg * L.gin_stage_bytes) + vox;  // gs[c * 64]
                tma::wait_parity(&gin_full[sg], (it / SG) & 1u, abort_flag, p.status, 23);
                tma::wait_parity(&d1_full[buf], (it >> 1) & 1u, abort_flag, p.status, 19);
                umma::fence_after_sync();
                const bool live = valid && !*abort_flag;
                const uint32_t d1 = tmem + kMmaD1Col + buf * 128 + ((uint32_t)(32 * warp) << 16);
                for (int c0 = 0; c0 < C16; c0 += 16) {
                    float acc[16];
                    umma::tmem_ld16(d1 + c0, acc);
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int c = c0 + i;
                        if (c < C) {
                            float v = gs[c * SV] + acc[i];
                            if (c == p.mask_channel && live) v = ip[(int64_t)c * p.in_sc] > 0.f ? v : 0.f;  // hand the layer below a gated gradient
                            if (live) gp[(int64_t)c * p.gi_sc] = v;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) tma::mbar_arrive(&gin_empty[sg]);
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) tma::mbar_arrive(&d1_empty[buf]);
            }
        }
        // ---- the weight gradient: D2[c][t] + D2[c][32 + t], one partial row per block ----
        tma::wait_parity(final_bar, 0, abort_flag, p.status, 20);
        umma::fence_after_sync();
        // M = 64: channel c sits in lane 32 (c / 16) + (c % 16); M = 128: in lane c
        const int ch = C <= 64 ? ((lane < 16) ? 16 * warp + lane : -1) : 32 * warp + lane;
        float d[64];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float part[16];
            umma::tmem_ld16(tmem + kMmaD2Col + 16 * q + ((uint32_t)(32 * warp) << 16), part);
#pragma unroll
            for (int i = 0; i < 16; ++i) d[16 * q + i] = part[i];
        }
        if (ch >= 0 && ch < C && !*abort_flag) {
            float *dst = p.part_k + (int64_t)blockIdx.x * C * TAPS + ch * TAPS;
#pragma unroll
            for (int t = 0; t < TAPS; ++t) dst[t] = d[t] + d[32 + t];
        }
        umma::fence_before_sync();
    }
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, kMmaTmemCols);
}

}  // namespace fast
}  // namespace msd

// Host side and instantiations of the TMA-staged 2D forward kernel (fast_forward_2d.cuh).
#include <cudaTypedefs.h>
#include <mutex>
#include <string.h>
#include "fast_forward_2d.cuh"

namespace msd {
namespace fast {

int sm_count(int device);

// ---- TMA descriptor cache ---------------------------------------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
    static std::once_flag once;
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
    });
    return fn;
}

struct MapKey {
    const void *ptr;
    int64_t dims[5], strides[5];
    int box[5];
    int rank, device, pad;  // explicit tail so that memcmp sees no padding
    bool operator==(const MapKey &o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapEntry {
    MapKey key;
    CUtensorMap map;
    bool used;
};
// Open-addressing hash table.  A block forward + backward of depth 100 touches about 500
// distinct descriptors (the channel count and the base pointer of the single-channel views
// change per layer); when the table is three quarters full it is simply emptied.
static const int kMapSlots = 4096;
static std::mutex g_map_mu;
static MapEntry *g_maps = nullptr;
static int g_map_count = 0;

static uint64_t hash_key(const MapKey &k) {
    const unsigned char *b = reinterpret_cast<const unsigned char *>(&k);
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i < sizeof(MapKey); ++i) h = (h ^ b[i]) * 1099511628211ull;
    return h;
}

// Tiled descriptor over a float32 tensor; dims/strides innermost first, strides in elements
// (strides[0] must be 1).  Descriptors are cached by (device, pointer, geometry, box).
// `swizzle128`: the box's 128-byte rows land with their 16-byte chunks XOR-permuted by the row
// index (the layout the tensor cores read); the innermost box extent must then be 32 floats.
int get_tensor_map(int device, const void *ptr, int rank, const int64_t *dims, const int64_t *strides, const int *box, CUtensorMap *out,
                   bool swizzle128) {
    MapKey key;
    memset(&key, 0, sizeof(key));
    key.ptr = ptr, key.rank = rank, key.device = device, key.pad = swizzle128 ? 1 : 0;
    for (int i = 0; i < rank; ++i) key.dims[i] = dims[i], key.strides[i] = strides[i], key.box[i] = box[i];
    const uint64_t h = hash_key(key);
    std::lock_guard<std::mutex> l(g_map_mu);
    if (!g_maps) g_maps = new MapEntry[kMapSlots]();
    int slot = (int)(h & (kMapSlots - 1));
    while (g_maps[slot].used) {
        if (g_maps[slot].key == key) {
            *out = g_maps[slot].map;
            return MSD_OK;
        }
        slot = (slot + 1) & (kMapSlots - 1);
    }
    PFN_cuTensorMapEncodeTiled_v12000 enc = get_encode();
    if (!enc) MSD_FAIL(MSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t gdim[5], gstr[4];
    cuuint32_t bdim[5], estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = (cuuint64_t)dims[i];
        bdim[i] = (cuuint32_t)box[i];
        estr[i] = 1;
        if (i > 0) gstr[i - 1] = (cuuint64_t)strides[i] * sizeof(float);
    }
    CUtensorMap m;
    CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void *>(ptr), gdim, gstr, bdim, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) MSD_FAIL(MSD_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (g_map_count >= kMapSlots * 3 / 4) {
        memset(g_maps, 0, sizeof(MapEntry) * kMapSlots);
        g_map_count = 0;
        slot = (int)(h & (kMapSlots - 1));
    }
    g_maps[slot].key = key;
    g_maps[slot].map = m;
    g_maps[slot].used = true;
    ++g_map_count;
    *out = m;
    return MSD_OK;
}

// ---- kernel variants ----------------------------------------------------------------------
template <int D, int R, int Q, int K, int NT, int TW>
static int launch_fwd2d(const CUtensorMap &map, const Fwd2dParams &p, int grid, int stages, cudaStream_t s) {
    using Cfg = Fwd2dCfg<D, R, Q, K, TW>;
    auto kern = forward2d_kernel<D, R, Q, K, NT, TW>;
    const size_t smem = 256 + (size_t)stages * Cfg::STAGE_BYTES + (size_t)((p.C * fwd_weight_floats(NT) + 31) & ~31) * 4;
    MSD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    MSD_CUDA_TRY(tma::launch_pdl(kern, dim3(grid), dim3(Cfg::THREADS), smem, s, map, p));
    return MSD_OK;
}

#define V(D, R, Q, K, NT, TW)                                                                                                   \
    {                                                                                                                           \
        launch_fwd2d<D, R, Q, K, NT, TW>, Fwd2dCfg<D, R, Q, K, TW>::THREADS, Fwd2dCfg<D, R, Q, K, TW>::TH, TW,                      \
            Fwd2dCfg<D, R, Q, K, TW>::BH, Fwd2dCfg<D, R, Q, K, TW>::BW, Fwd2dCfg<D, R, Q, K, TW>::STAGE_BYTES                     \
    }
// 2D, per dilation (index D-1).  Tile = (Q*R*D) rows x TW columns:
//   variant 0: 4-row lattice, 4 column segments per thread, 128 columns
//   variant 1: 4-row lattice, 2 segments (twice the warps), 128 columns
//   variant 2: 6-row lattice, 4 segments, 128 columns
//   variant 3: 4-row lattice, 2 segments, 64 columns (twice the tiles: finer load balance)
//   variant 4: 3-row lattice, taller stacks (Q chosen for 36..48 rows), 4 segments, 128 columns
//   variant 5: 8-row lattice (fewest shared loads per FMA), 4 segments, 128 columns
//   variant 6: 6-row lattice, 2 segments (twice the warps), 128 columns
//   variant 7: tiles of 60..64 rows with ONE row stack where the dilation allows (lattices of 6..15
//              rows: the taller the lattice, the fewer shared loads per FMA), 4 segments
//   variant 8: the same with 2 segments (twice the warps)
static const int kNumFwd2dVariants = 9;
static const Fwd2dVariant kFwd2d[10][kNumFwd2dVariants] = {
    {V(1, 4, 8, 4, 1, 128), V(1, 4, 8, 2, 1, 128), V(1, 6, 8, 4, 1, 128), V(1, 4, 8, 2, 1, 64), V(1, 3, 14, 4, 1, 128), V(1, 8, 8, 4, 1, 128), V(1, 6, 8, 2, 1, 128), V(1, 15, 4, 4, 1, 128), V(1, 15, 4, 2, 1, 128)},
    {V(2, 4, 4, 4, 1, 128), V(2, 4, 4, 2, 1, 128), V(2, 6, 4, 4, 1, 128), V(2, 4, 4, 2, 1, 64), V(2, 3, 7, 4, 1, 128), V(2, 8, 4, 4, 1, 128), V(2, 6, 4, 2, 1, 128), V(2, 15, 2, 4, 1, 128), V(2, 15, 2, 2, 1, 128)},
    {V(3, 4, 3, 4, 1, 128), V(3, 4, 3, 2, 1, 128), V(3, 6, 3, 4, 1, 128), V(3, 4, 3, 2, 1, 64), V(3, 3, 5, 4, 1, 128), V(3, 8, 2, 4, 1, 128), V(3, 6, 3, 2, 1, 128), V(3, 10, 2, 4, 1, 128), V(3, 10, 2, 2, 1, 128)},
    {V(4, 4, 2, 4, 1, 128), V(4, 4, 2, 2, 1, 128), V(4, 6, 2, 4, 1, 128), V(4, 4, 2, 2, 1, 64), V(4, 3, 4, 4, 1, 128), V(4, 8, 2, 4, 1, 128), V(4, 6, 2, 2, 1, 128), V(4, 15, 1, 4, 1, 128), V(4, 15, 1, 2, 1, 128)},
    {V(5, 4, 2, 4, 1, 128), V(5, 4, 2, 2, 1, 128), V(5, 6, 2, 4, 1, 128), V(5, 4, 2, 2, 1, 64), V(5, 3, 3, 4, 1, 128), V(5, 8, 1, 4, 1, 128), V(5, 6, 1, 2, 1, 128), V(5, 12, 1, 4, 1, 128), V(5, 12, 1, 2, 1, 128)},
    {V(6, 4, 2, 4, 1, 128), V(6, 4, 2, 2, 1, 128), V(6, 6, 2, 4, 1, 128), V(6, 4, 2, 2, 1, 64), V(6, 3, 2, 4, 1, 128), V(6, 8, 1, 4, 1, 128), V(6, 6, 1, 2, 1, 128), V(6, 10, 1, 4, 1, 128), V(6, 10, 1, 2, 1, 128)},
    {V(7, 4, 2, 4, 1, 128), V(7, 4, 2, 2, 1, 128), V(7, 6, 1, 4, 1, 128), V(7, 4, 2, 2, 1, 64), V(7, 3, 2, 4, 1, 128), V(7, 8, 1, 4, 1, 128), V(7, 6, 1, 2, 1, 128), V(7, 9, 1, 4, 1, 128), V(7, 9, 1, 2, 1, 128)},
    {V(8, 4, 1, 4, 1, 128), V(8, 4, 1, 2, 1, 128), V(8, 6, 1, 4, 1, 128), V(8, 4, 1, 2, 1, 64), V(8, 3, 2, 4, 1, 128), V(8, 8, 1, 4, 1, 128), V(8, 6, 1, 2, 1, 128), V(8, 8, 1, 4, 1, 128), V(8, 8, 1, 2, 1, 128)},
    {V(9, 4, 1, 4, 1, 128), V(9, 4, 1, 2, 1, 128), V(9, 6, 1, 4, 1, 128), V(9, 4, 1, 2, 1, 64), V(9, 3, 1, 4, 1, 128), V(9, 8, 1, 4, 1, 128), V(9, 6, 1, 2, 1, 128), V(9, 7, 1, 4, 1, 128), V(9, 7, 1, 2, 1, 128)},
    {V(10, 4, 1, 4, 1, 128), V(10, 4, 1, 2, 1, 128), V(10, 6, 1, 4, 1, 128), V(10, 4, 1, 2, 1, 64), V(10, 3, 1, 4, 1, 128), V(10, 8, 1, 4, 1, 128), V(10, 6, 1, 2, 1, 128), V(10, 6, 1, 4, 1, 128), V(10, 6, 1, 2, 1, 128)},
};
// 3D (three z-taps per staged plane), per dilation: variant 0 = 4-row lattice, 4 column
// segments per thread; variant 1 = 4-row lattice, 2 segments (twice the warps, shorter tiles
// where the block would otherwise exceed ~500 threads and run out of registers); variant 2 =
// variant 0 with more row stacks for the small dilations (12-13 compute warps instead of 8-9:
// the kernel is bound by FP32 issue, and more resident warps hide its shared-memory latency);
// variant 3 = 8-row lattice, 2 segments (dilations up to 6; 4 segments for 7 and 8; a 6-row
// lattice with 4 segments for 9 and 10): per packed FMA fewer shared loads and fewer instructions
// that fetch and duplicate the 27 weights (measured: 0 - 3 % faster than variant 0; a 6-row
// lattice with 4 segments for the small dilations was 10 % slower).
static const int kNumFwd3dVariants = 4;
static const Fwd2dVariant kFwd3d[10][kNumFwd3dVariants] = {
    {V(1, 4, 8, 4, 3, 128), V(1, 4, 6, 2, 3, 128), V(1, 4, 13, 4, 3, 128), V(1, 8, 4, 2, 3, 128)},
    {V(2, 4, 4, 4, 3, 128), V(2, 4, 3, 2, 3, 128), V(2, 4, 6, 4, 3, 128), V(2, 8, 2, 2, 3, 128)},
    {V(3, 4, 3, 4, 3, 128), V(3, 4, 2, 2, 3, 128), V(3, 4, 4, 4, 3, 128), V(3, 8, 1, 2, 3, 128)},
    {V(4, 4, 2, 4, 3, 128), V(4, 4, 1, 2, 3, 128), V(4, 4, 3, 4, 3, 128), V(4, 8, 1, 2, 3, 128)},
    {V(5, 4, 2, 4, 3, 128), V(5, 4, 1, 2, 3, 128), V(5, 4, 2, 4, 3, 128), V(5, 8, 1, 2, 3, 128)},
    {V(6, 4, 2, 4, 3, 128), V(6, 4, 1, 2, 3, 128), V(6, 4, 2, 4, 3, 128), V(6, 8, 1, 2, 3, 128)},
    {V(7, 4, 2, 4, 3, 128), V(7, 4, 1, 2, 3, 128), V(7, 4, 2, 4, 3, 128), V(7, 8, 1, 4, 3, 128)},
    {V(8, 4, 1, 4, 3, 128), V(8, 4, 1, 2, 3, 128), V(8, 4, 1, 4, 3, 128), V(8, 8, 1, 4, 3, 128)},
    {V(9, 4, 1, 4, 3, 128), V(9, 4, 1, 2, 3, 128), V(9, 4, 1, 4, 3, 128), V(9, 6, 1, 4, 3, 128)},
    {V(10, 4, 1, 4, 3, 128), V(10, 4, 1, 2, 3, 128), V(10, 4, 1, 4, 3, 128), V(10, 6, 1, 4, 3, 128)},
};
#undef V

static const size_t kFwdSmemBudget = 220 * 1024;

int num_variants(int family) {
    switch (family) {
        case FWD2D: return kNumFwd2dVariants;  // lattice rows x column segments x tile width
        case BWD2D: return 3;  // 4 / 8 voxels per thread / X warps + K warps
        case FWD3D: return kNumFwd3dVariants;  // 4 / 2 column segments per thread / more row stacks
        case BWD3D: return 3;  // unsplit consumers / X warps + K warps / tensor cores
        default: return 1;
    }
}

static bool fwd_plan(const View &in, int nd, int d, const Fwd2dVariant **var, int *stages) {
    if (d < 1 || d > 10) return false;
    const int wp = fwd_weight_floats(nd == 3 ? 3 : 1);
    const int nvar = nd == 3 ? kNumFwd3dVariants : kNumFwd2dVariants;
    int v = tuning_get(nd == 3 ? FWD3D : FWD2D, d);
    // untuned 2D: the variants that won on a large image (16 x 1024 x 1024, where the number of
    // tiles per SM does not matter); the autotuner refines this per shape
    static const int kFwd2dDefault[10] = {5, 5, 6, 5, 2, 2, 8, 8, 8, 6};
    if (v < 0 || v >= nvar) v = nd == 3 ? 0 : (in.x <= 64 ? 3 : kFwd2dDefault[d - 1]);  // narrow images: the 64-column tiles
    const Fwd2dVariant *cand = nd == 3 ? &kFwd3d[d - 1][v] : &kFwd2d[d - 1][v];
    const size_t fixed = 256 + (size_t)((in.c * wp + 31) & ~31) * 4;
    if (fixed + 2 * (size_t)cand->stage_bytes > kFwdSmemBudget) {
        cand = nd == 3 ? &kFwd3d[d - 1][0] : &kFwd2d[d - 1][0];
        if (fixed + 2 * (size_t)cand->stage_bytes > kFwdSmemBudget) return false;
    }
    int s = (int)((kFwdSmemBudget - fixed) / cand->stage_bytes);
    if (s > kFwdMaxStages) s = kFwdMaxStages;
    *var = cand;
    *stages = s;
    return true;
}

size_t forward_workspace_bytes(int nd, int64_t voxels) { return nd == 3 ? (size_t)voxels * 3 * sizeof(float) + 256 : 0; }

bool forward_supported(const View &in, const View &out, int nd, int d, const void *ws, size_t wsb) {
    if (out.c != 1 || in.c < 1 || in.c > 4096) return false;
    if (in.sx != 1 || out.sx != 1) return false;
    // TMA: 16-byte aligned base and strides
    if ((in.sy % 4) || (in.sz % 4) || (in.sc % 4) || (in.sn % 4) || (((uintptr_t)in.p) & 15)) return false;
    if (in.x < 16 || in.x >= (1LL << 31) || in.y >= (1LL << 31) || in.z >= (1LL << 31)) return false;
    if (in.sy < in.x) return false;
    if (nd == 3) {
        // the z-gather kernel writes 128-bit vectors and needs the scratch planes
        if ((in.x % 4) || (out.sy % 4) || (out.sz % 4) || (out.sn % 4) || (((uintptr_t)out.p) & 15)) return false;
        if (!ws || wsb < forward_workspace_bytes(3, in.n * in.z * in.y * in.x)) return false;
    }
    const Fwd2dVariant *var;
    int stages;
    return fwd_plan(in, nd, d, &var, &stages);
}

int forward(bool relu, const View &in, const float *k, const float *bias, const View &out, int nd, int d, void *ws, size_t wsb, int device,
               cudaStream_t s) {
    const Fwd2dVariant *var;
    int stages;
    if (!fwd_plan(in, nd, d, &var, &stages)) MSD_FAIL(MSD_ERR_UNSUPPORTED, "forward: shape not supported");
    CUtensorMap map;
    int rc;
    if (nd == 3) {
        const int64_t dims[5] = {in.x, in.y, in.z, in.c, in.n};
        const int64_t strides[5] = {1, in.sy, in.sz, in.sc, in.sn};
        const int box[5] = {var->bw, var->bh, 1, 1, 1};
        rc = get_tensor_map(device, in.p, 5, dims, strides, box, &map, false);
    } else {
        const int64_t dims[4] = {in.x, in.y, in.c, in.n};
        const int64_t strides[4] = {1, in.sy, in.sc, in.sn};
        const int box[4] = {var->bw, var->bh, 1, 1};
        rc = get_tensor_map(device, in.p, 4, dims, strides, box, &map, false);
    }
    if (rc) return rc;
    Fwd2dParams p;
    memset(&p, 0, sizeof(p));
    const int64_t vox = in.n * in.z * in.y * in.x;
    if (nd == 3) {
        p.out = (float *)ws;  // u[3][N][Z][Y][X]
        p.out_st = vox, p.out_sn = in.z * in.y * in.x, p.out_sz = in.y * in.x, p.out_sy = in.x;
    } else {
        p.out = (float *)out.p;
        p.out_st = 0, p.out_sn = out.sn, p.out_sz = 0, p.out_sy = out.sy;
    }
    p.k = k, p.bias = bias;
    p.N = (int)in.n, p.C = (int)in.c, p.Z = (int)in.z, p.Y = (int)in.y, p.X = (int)in.x;
    get_z_window((int)in.z, &p.z0, &p.ZW);
    const int gather_z0 = p.z0, gather_zw = p.ZW;
    const int phase = nd == 3 ? get_forward_phase() : FWD_BOTH;
    if (nd == 3 && phase == FWD_BOTH) {
        // the z-gather of plane z reads the partial sums of planes z - d and z + d: compute
        // those for the window widened by d on both sides (clipped to the local buffer)
        const int lo = p.z0 - d < 0 ? 0 : p.z0 - d;
        const int hi = p.z0 + p.ZW + d > (int)in.z ? (int)in.z : p.z0 + p.ZW + d;
        p.z0 = lo, p.ZW = hi - lo;
    }
    p.tiles_x = (int)ceil_div(in.x, var->tw);
    p.tiles_y = (int)ceil_div(in.y, var->th);
    p.num_tiles = (long long)p.tiles_x * p.tiles_y * p.ZW * in.n;
    p.stages = stages;
    p.relu = relu ? 1 : 0;
    p.status = tma::device_status_ptr(device);
    if (!p.status) MSD_FAIL(MSD_ERR_CUDA, "forward: cannot locate the device status word");
    if (phase != FWD_GATHER_ONLY) {
        int grid = sm_count(device);
        if (p.num_tiles < grid) grid = (int)p.num_tiles;
        rc = var->launch(map, p, grid, stages, s);
        if (rc) return rc;
        count_launch(true);
    }
    if (nd == 3 && phase != FWD_SUMS_ONLY) {
        const int64_t quads = in.n * (int64_t)gather_zw * in.y * in.x / 4;
        int64_t g = ceil_div(quads, 256);
        const int64_t gmax = (int64_t)sm_count(device) * 16;
        if (g > gmax) g = gmax;
        zgather_kernel<<<(unsigned)g, 256, 0, s>>>((const float *)ws, (float *)out.p, out.sn, out.sz, out.sy, bias, (int)in.n, (int)in.z, (int)in.y,
                                                   (int)in.x, gather_z0, gather_zw, d, relu ? 1 : 0);
        count_launch(true);
        MSD_CUDA_TRY(cudaGetLastError());
    }
    return MSD_OK;
}

}  // namespace fast
}  // namespace msd

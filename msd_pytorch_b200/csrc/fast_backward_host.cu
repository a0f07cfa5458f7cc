// Host side of the fused backward: eligibility, shared-memory budget, launch, second pass.
#include <mutex>
#include "fast_backward.cuh"

namespace msd {
namespace generic {
int reduce_partials_f32(const float *partial, int nparts, int64_t pitch, int64_t nout, float *dst, cudaStream_t s);
}
namespace fast {

int get_tensor_map(int device, const void *ptr, int rank, const int64_t *dims, const int64_t *strides, const int *box, CUtensorMap *out,
                   bool swizzle128 = false);
extern BwdLaunchFn bwd3d_hybrid_launcher;
size_t bwd3d_hybrid_smem(int C, int Dp, int stages);
extern BwdLaunchFn bwd2d_launchers[2][2][3];
extern BwdLaunchFn bwd3d_launchers[2][3];
extern BwdLaunchFn bwd3d_split_launcher;
extern BwdLaunchFn bwd2d_split_launcher;


static const int kMaxFastDilation = 16;
static const size_t kSmemBudget = 220 * 1024;
static const int kMaxGrid = 320;

int sm_count(int device) {
    static std::mutex mu;
    static int cache[64] = {0};
    if (device < 0 || device >= 64) return 148;
    std::lock_guard<std::mutex> l(mu);
    if (!cache[device]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0) v = 148;
        cache[device] = v;
    }
    return cache[device];
}

static bool aligned_view(const View *v) {
    if (!v) return true;
    if (v->sy < v->x || v->x >= (1LL << 31) || v->y >= (1LL << 31) || v->z >= (1LL << 31)) return false;
    return v->sx == 1 && (v->sn % 4) == 0 && (v->sc % 4) == 0 && (v->sy % 4) == 0 && (v->sz % 4) == 0 && (((uintptr_t)v->p) & 15) == 0;
}

struct BwdPlan {
    int txq16, j, stages, blocks_per_sm;
    size_t smem;
    bool split;  // kernel with X warps and K warps (fast_backward_split.cuh)
    bool mma;    // 3D kernel with the input gradient on the tensor cores (fast_backward3d_hybrid.cuh)
};

// geometry of the role-split 3D kernel (the constants of the same names there)
static const int kSplitKWarps = 8, kSplitMaxDilation = 12, kSplitMaxStages = 8, kSplitHeader = 512;
static int split_rows(int nd) { return nd == 3 ? 4 : 8; }  // rows per tile
static int split_cb(int nd) { return nd == 3 ? 4 : 2; }    // channels per ring stage
// below this many input channels the per-tile set-up of the split kernel outweighs its faster
// channel loop (large dilations have more border tiles, whose set-up reads global memory)
static int split_min_channels(int d) { return d <= 5 ? 8 : 10; }
// tensor-core kernel (fast_backward3d_hybrid.cuh): rows per tile, channels per ring stage, most ring stages, fewest channels
static const int kMmaRowsHost = 2, kMmaCBHost = 8, kMmaMaxStagesHost = 8, kMmaMinChannels = 8;

static bool plan(const BackwardArgs &a, BwdPlan *pl) {
    const View &g = *a.gout;
    const int nd = a.nd;
    const int64_t C = a.gin ? a.gin->c : a.in->c;
    const int RT = nd == 3 ? 9 : 3, TAPS_PAD = nd == 3 ? 28 : 12;
    const bool do_x = a.gin != nullptr, do_k = a.gk != nullptr;
    const int Dp = (a.d + 3) & ~3;
    pl->txq16 = g.x <= 64 ? 1 : 0;
    pl->split = false;
    pl->mma = false;
    if (nd == 3 && do_x && do_k && !a.out && (g.x % 128) == 0 && a.d <= kSplitMaxDilation && C >= kMmaMinChannels && C <= 128 &&
        tuning_get(BWD3D, a.d) == 2) {
        // tensor-core kernel: tiles of 2 rows x 128 columns, ring stages of 8 channels
        for (int s = kMmaMaxStagesHost; s >= 3; --s) {
            const size_t need = bwd3d_hybrid_smem((int)C, Dp, s);
            if (need <= (size_t)227 * 1024) {
                pl->j = 1, pl->stages = s, pl->blocks_per_sm = 1, pl->smem = need, pl->mma = true;
                return true;
            }
        }
    }
    const int TX = pl->txq16 ? 64 : 128;
    const bool split3d = nd == 3 && C >= split_min_channels(a.d) && tuning_get(BWD3D, a.d) != 0;
    const bool split2d = nd == 2 && tuning_get(BWD2D, a.d) == 2;
    if ((split3d || split2d) && do_x && do_k && (g.x % 128) == 0 && a.d <= kSplitMaxDilation) {
        // role-split kernel: 4 X warps + 8 K warps on tiles of 4 (2D: 8) rows x 128 columns, 4 (2)
        // channels per ring stage; the table of M (27 or 9 taps x (rows x 128 + 4) floats) beside the (double-buffered) halo rows
        const int TR = split_rows(nd), TXP = 128 + 2 * Dp;
        const size_t halo = 2 * (size_t)RT * ((TR * TXP + 31) & ~31) * (a.out ? 2 : 1) + ((3 * RT * (TR * 128 + 4) + 31) & ~31);  // two halo buffers + the table
        const size_t fixed = kSplitHeader + (size_t)4 * (C * TAPS_PAD + (size_t)kSplitKWarps * C * TAPS_PAD + halo);
        const size_t stage = (size_t)4 * 2 * split_cb(nd) * TR * 128;
        if (fixed + 2 * stage <= kSmemBudget) {
            int s = (int)((kSmemBudget - fixed) / stage);
            if (s > kSplitMaxStages) s = kSplitMaxStages;
            pl->j = 1, pl->stages = s, pl->blocks_per_sm = 1, pl->smem = fixed + (size_t)s * stage, pl->split = true;
            return true;
        }
    }
    int j = 1;
    if (nd == 2) {
        const int tuned = tuning_get(BWD2D, a.d);
        j = tuned == 0 ? 1 : 2;  // variant 0: 4 voxels per thread, variant 1 (default): 8
    }
    for (; j >= 1; --j) {
        const int ncw = bwd_consumer_warps(nd);
        const int TR = (ncw * 32 / (TX / 4)) * j;
        const size_t halo = (size_t)RT * (((int64_t)TR * (TX + 2 * Dp) + 31) & ~31) * (a.out ? 2 : 1);
        const size_t fixed = 256 + (size_t)4 * ((do_x ? C * TAPS_PAD : 0) + (do_k ? ncw * C * TAPS_PAD : 0) + halo);
        const size_t stage = (size_t)4 * ((do_x ? 1 : 0) + (do_k ? 1 : 0)) * TR * TX;
        // two resident blocks per SM for the small 2D variant when both fit
        int bps = (nd == 2 && j == 1) ? 2 : 1;
        size_t budget = bps == 2 ? (size_t)110 * 1024 : kSmemBudget;
        if (bps == 2 && fixed + 3 * stage > budget) {
            bps = 1;
            budget = kSmemBudget;
        }
        if (fixed + 2 * stage > budget) continue;
        int s = (int)((budget - fixed) / stage);
        if (s > kMaxStages) s = kMaxStages;
        pl->j = j;
        pl->stages = s;
        pl->blocks_per_sm = bps;
        pl->smem = fixed + (size_t)s * stage;
        return true;
    }
    return false;
}

bool backward_supported(const BackwardArgs &a) {
    if (!a.gout || a.gout->c != 1) return false;
    if (!a.gin && !a.gk) return false;  // bias alone goes through the generic reduction
    if (a.gin && !a.k) return false;
    if (a.gk && !a.in) return false;
    if (a.d < 1 || a.d > kMaxFastDilation) return false;
    const View &g = *a.gout;
    if ((g.x % 4) != 0 || g.x < 16) return false;
    if (!aligned_view(a.gout) || !aligned_view(a.out) || !aligned_view(a.in) || !aligned_view(a.gin)) return false;
    const int64_t C = a.gin ? a.gin->c : a.in->c;
    if (C < 1 || C > 4096) return false;
    if (g.n * g.z > (1LL << 40)) return false;
    BwdPlan pl;
    if (!plan(a, &pl)) return false;
    if (a.gk || a.gb) {
        if (!a.ws || a.wsb < backward_workspace_bytes(a.nd, C)) return false;
    }
    return true;
}

size_t backward_workspace_bytes(int nd, int64_t c_in) {
    const int taps = nd == 3 ? 27 : 9;
    return (size_t)kMaxGrid * (c_in * taps + 64) * sizeof(float) + 512;
}

struct ReduceTable {
    ReduceEntry e[ReduceList::kMax];
};

// Pass two for a table of layers: dst[j] += sum over the blocks' partials, block order fixed.
__global__ void __launch_bounds__(128) reduce_table_kernel(const __grid_constant__ ReduceTable t) {
    const ReduceEntry &e = t.e[blockIdx.y];
    const int j = blockIdx.x * 128 + threadIdx.x;
    const int nk = (e.pk && e.gk) ? e.nk : 0;
    const int64_t pitch = e.pitch ? e.pitch : nk, pitch_b = e.pitch_b ? e.pitch_b : 1;
    if (j < nk) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        int q = 0;
        for (; q + 3 < e.nparts; q += 4) {
            s0 += e.pk[(int64_t)(q + 0) * pitch + j];
            s1 += e.pk[(int64_t)(q + 1) * pitch + j];
            s2 += e.pk[(int64_t)(q + 2) * pitch + j];
            s3 += e.pk[(int64_t)(q + 3) * pitch + j];
        }
        for (; q < e.nparts; ++q) s0 += e.pk[(int64_t)q * pitch + j];
        e.gk[j] += (s0 + s1) + (s2 + s3);
    } else if (j == nk && e.pb && e.gb) {
        float s0 = 0.f;
        for (int q = 0; q < e.nparts; ++q) s0 += e.pb[(int64_t)q * pitch_b];
        e.gb[0] += s0;
    }
}

int flush_reductions(ReduceList *list, cudaStream_t s) {
    if (!list || list->count == 0) return MSD_OK;
    ReduceTable t;
    int max_n = 1;
    for (int i = 0; i < list->count; ++i) {
        t.e[i] = list->e[i];
        const int n = ((list->e[i].pk && list->e[i].gk) ? list->e[i].nk : 0) + 1;
        if (n > max_n) max_n = n;
    }
    dim3 grid((unsigned)ceil_div(max_n, 128), (unsigned)list->count);
    reduce_table_kernel<<<grid, 128, 0, s>>>(t);
    count_launch(false);
    list->count = 0;
    list->ws_used = 0;
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

// g = (a > 0) ? g : 0 on one channel (both views [N,1,Z,Y,X] with unit x-stride, X % 4 == 0):
// gates the top gradient channel once before a block's backward, so that every layer's kernel
// can read an already gated gradient.
__global__ void __launch_bounds__(256)
gate_channel_kernel(float *__restrict__ g, int64_t g_sn, int64_t g_sz, int64_t g_sy, const float *__restrict__ a, int64_t a_sn, int64_t a_sz,
                    int64_t a_sy, int N, int Z, int Y, int X) {
    const int xq = X / 4;
    const int64_t total = (int64_t)N * Z * Y * xq;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int x4 = (int)(i % xq);
        int64_t r = i / xq;
        const int y = (int)(r % Y);
        r /= Y;
        const int z = (int)(r % Z), n = (int)(r / Z);
        float4 *gp = reinterpret_cast<float4 *>(g + n * g_sn + z * g_sz + (int64_t)y * g_sy + 4 * x4);
        const float4 av = *reinterpret_cast<const float4 *>(a + n * a_sn + z * a_sz + (int64_t)y * a_sy + 4 * x4);
        float4 gv = *gp;
        gv.x = av.x > 0.f ? gv.x : 0.f;
        gv.y = av.y > 0.f ? gv.y : 0.f;
        gv.z = av.z > 0.f ? gv.z : 0.f;
        gv.w = av.w > 0.f ? gv.w : 0.f;
        *gp = gv;
    }
}

bool gate_channel_supported(const View &g, const View &a) {
    return g.c == 1 && a.c == 1 && aligned_view(&g) && aligned_view(&a) && (g.x % 4) == 0 && g.n == a.n && g.z == a.z && g.y == a.y && g.x == a.x;
}

int gate_channel(const View &g, const View &a, int device, cudaStream_t s) {
    const int64_t quads = g.n * g.z * g.y * (g.x / 4);
    if (quads == 0) return MSD_OK;
    int64_t grid = ceil_div(quads, 256);
    const int64_t gmax = (int64_t)sm_count(device) * 16;
    if (grid > gmax) grid = gmax;
    gate_channel_kernel<<<(unsigned)grid, 256, 0, s>>>((float *)g.p, g.sn, g.sz, g.sy, (const float *)a.p, a.sn, a.sz, a.sy, (int)g.n, (int)g.z,
                                                      (int)g.y, (int)g.x);
    count_launch(true);
    MSD_CUDA_TRY(cudaGetLastError());
    return MSD_OK;
}

int backward(const BackwardArgs &a, int device, cudaStream_t s) {
    BwdPlan pl;
    if (!plan(a, &pl)) MSD_FAIL(MSD_ERR_UNSUPPORTED, "fused backward: shape not supported");
    const View &g = *a.gout;
    const bool do_x = a.gin != nullptr, do_k = a.gk != nullptr;
    const int64_t C = do_x ? a.gin->c : a.in->c;
    const int taps = a.nd == 3 ? 27 : 9;
    BwdParams p;
    memset(&p, 0, sizeof(p));
    if (a.out) {
        p.out = (const float *)a.out->p;
        p.out_sn = a.out->sn, p.out_sz = a.out->sz, p.out_sy = a.out->sy;
    }
    p.gout = (const float *)g.p;
    p.go_sn = g.sn, p.go_sz = g.sz, p.go_sy = g.sy;
    if (do_k) {
        p.in = (const float *)a.in->p;
        p.in_sn = a.in->sn, p.in_sc = a.in->sc, p.in_sz = a.in->sz, p.in_sy = a.in->sy;
    }
    if (do_x) {
        p.gin = (float *)a.gin->p;
        p.gi_sn = a.gin->sn, p.gi_sc = a.gin->sc, p.gi_sz = a.gin->sz, p.gi_sy = a.gin->sy;
    }
    p.k = a.k;
    p.N = (int)g.n, p.C = (int)C, p.Z = (int)g.z, p.Y = (int)g.y, p.X = (int)g.x;
    p.d = a.d, p.Dp = (a.d + 3) & ~3;
    const int TX = pl.txq16 ? 64 : 128;
    const int TR = pl.mma ? kMmaRowsHost : pl.split ? split_rows(a.nd) : (bwd_consumer_warps(a.nd) * 32 / (TX / 4)) * pl.j;
    get_z_window((int)g.z, &p.z0, &p.ZW);
    p.tiles_x = (int)ceil_div(g.x, TX);
    p.tiles_y = (int)ceil_div(g.y, TR);
    p.num_tiles = (long long)p.tiles_x * p.tiles_y * p.ZW * g.n;
    p.stages = pl.stages;
    p.mask_channel = (do_x && do_k) ? a.mask_channel : -1;
    p.status = tma::device_status_ptr(device);
    if (!p.status) MSD_FAIL(MSD_ERR_CUDA, "fused backward: cannot locate the device status word");
    int grid = sm_count(device) * pl.blocks_per_sm;
    if (grid > kMaxGrid) grid = kMaxGrid;
    if (p.num_tiles < grid) grid = (int)p.num_tiles;
    const bool do_b = a.gb != nullptr;
    const size_t need_k = do_k ? (((size_t)grid * C * taps * sizeof(float) + 255) & ~(size_t)255) : 0;
    const size_t need = need_k + (do_b ? (((size_t)grid * sizeof(float) + 255) & ~(size_t)255) : 0);
    if (a.defer && (a.defer->count == ReduceList::kMax || a.defer->ws_used + need > a.wsb)) {
        int rcf = flush_reductions(a.defer, s);
        if (rcf) return rcf;
    }
    if (need > a.wsb) MSD_FAIL(MSD_ERR_WORKSPACE, "fused backward: workspace of %zu bytes needed, %zu given", need, a.wsb);
    char *ws = (char *)a.ws + (a.defer ? a.defer->ws_used : 0);
    if (do_k) p.part_k = (float *)ws;
    if (do_b) p.part_b = (float *)(ws + need_k);
    // TMA descriptors: the two streamed tensors (a missing one aliases the other and is never
    // used) and the halo rows of gout / out (out aliases gout when there is no gate).
    CUtensorMap maps[4];
    {
        const int rank = a.nd == 3 ? 5 : 4;
        const View *views[4] = {do_k ? a.in : a.gin, do_x ? a.gin : a.in, a.gout, a.out ? a.out : a.gout};
        for (int which = 0; which < 4; ++which) {
            const View *v = views[which];
            if (pl.mma && which == 3) {  // the tensor-core kernel needs no gate halo
                maps[which] = maps[0];
                continue;
            }
            if (pl.mma && which == 1) {  // L2 prefetch box of the gradients: a whole tile of 64 channels
                const int64_t dims[5] = {v->x, v->y, v->z, v->c, v->n}, strides[5] = {1, v->sy, v->sz, v->sc, v->sn};
                const int box[5] = {TX, TR, 1, 64, 1};
                int rc2 = get_tensor_map(device, v->p, 5, dims, strides, box, &maps[1]);
                if (rc2) return rc2;
                continue;
            }
            const int cbox = (which < 2) ? (pl.split ? split_cb(a.nd) : pl.mma ? kMmaCBHost : 1) : 1;  // channels per box
            int box[5] = {which < 2 ? TX : TX + 2 * p.Dp, TR, a.nd == 3 ? 1 : cbox, a.nd == 3 ? cbox : 1, 1};
            int64_t dims[5], strides[5];
            if (a.nd == 3) {
                dims[0] = v->x, dims[1] = v->y, dims[2] = v->z, dims[3] = v->c, dims[4] = v->n;
                strides[0] = 1, strides[1] = v->sy, strides[2] = v->sz, strides[3] = v->sc, strides[4] = v->sn;
            } else {
                dims[0] = v->x, dims[1] = v->y, dims[2] = v->c, dims[3] = v->n, dims[4] = 1;
                strides[0] = 1, strides[1] = v->sy, strides[2] = v->sc, strides[3] = v->sn, strides[4] = 0;
            }
            int rc2 = get_tensor_map(device, v->p, rank, dims, strides, box, &maps[which]);
            if (rc2) return rc2;
        }
    }
    const int mode = do_x && do_k ? 2 : (do_k ? 1 : 0);
    BwdLaunchFn fn = a.nd == 3 ? (pl.mma ? bwd3d_hybrid_launcher : pl.split ? bwd3d_split_launcher : bwd3d_launchers[pl.txq16][mode])
                               : (pl.split ? bwd2d_split_launcher : bwd2d_launchers[pl.txq16][pl.j - 1][mode]);
    int rc = fn(maps, p, grid, pl.smem, s);
    if (rc) return rc;
    count_launch(true);
    if (pl.split) count_split_launch();
    if (pl.mma) count_mma_launch();
    if (do_k || do_b) {
        ReduceList single;
        ReduceList *list = a.defer ? a.defer : &single;
        if (!a.defer) single.count = 0, single.ws_used = 0;
        ReduceEntry &e = list->e[list->count++];
        e.pk = p.part_k, e.pb = p.part_b, e.gk = a.gk, e.gb = a.gb, e.nparts = grid, e.nk = (int)(C * taps);
        e.pitch = 0, e.pitch_b = 0;
        list->ws_used += need;
        if (!a.defer && (rc = flush_reductions(list, s))) return rc;
    }
    return MSD_OK;
}

}  // namespace fast
}  // namespace msd

// Host side of the fused backward: eligibility, shared-memory budget, launch, second pass.
#include <mutex>
#include "fast_backward.cuh"

namespace msd {
namespace generic {
int reduce_partials_f32(const float *partial, int nparts, int64_t pitch, int64_t nout, float *dst, cudaStream_t s);
}
namespace fast {

extern BwdLaunchFn bwd2d_launchers[2][2][3];
extern BwdLaunchFn bwd3d_launchers[2][3];

static const int kMaxFastDilation = 16;
static const size_t kSmemBudget = 200 * 1024;
static const int kMaxGrid = 148 * 4;

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
    return v->sx == 1 && (v->sn % 4) == 0 && (v->sc % 4) == 0 && (v->sy % 4) == 0 && (v->sz % 4) == 0 && (((uintptr_t)v->p) & 15) == 0;
}

struct BwdPlan {
    int txq16, j, stages;
    size_t smem;
};

static bool plan(const BackwardArgs &a, BwdPlan *pl) {
    const View &g = *a.gout;
    const int nd = a.nd;
    const int64_t C = a.gin ? a.gin->c : a.in->c;
    const int RT = nd == 3 ? 9 : 3, TAPS_PAD = nd == 3 ? 28 : 12;
    const bool do_x = a.gin != nullptr, do_k = a.gk != nullptr;
    const int Dp = (a.d + 3) & ~3;
    pl->txq16 = g.x <= 64 ? 1 : 0;
    const int TX = pl->txq16 ? 64 : 128;
    int j = 1;
    if (nd == 2) {
        const int tuned = tuning_get(BWD2D, a.d);
        j = tuned == 0 ? 1 : 2;  // variant 0: 4 voxels per thread, variant 1 (default): 8
    }
    for (; j >= 1; --j) {
        const int TR = (kConsumers / (TX / 4)) * j;
        const size_t fixed = 256 + (size_t)4 * ((do_x ? C * TAPS_PAD : 0) + (do_k ? kConsumerWarps * C * TAPS_PAD : 0) +
                                                 (int64_t)RT * TR * (TX + 2 * Dp));
        const size_t stage = (size_t)4 * ((do_x ? 1 : 0) + (do_k ? 1 : 0)) * TR * TX;
        if (fixed + 2 * stage > kSmemBudget) continue;
        int s = (int)((kSmemBudget - fixed) / stage);
        if (s > kMaxStages) s = kMaxStages;
        pl->j = j;
        pl->stages = s;
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
    const int TR = (kConsumers / (TX / 4)) * pl.j;
    p.tiles_x = (int)ceil_div(g.x, TX);
    p.tiles_y = (int)ceil_div(g.y, TR);
    p.num_tiles = (long long)p.tiles_x * p.tiles_y * g.z * g.n;
    p.stages = pl.stages;
    p.status = tma::device_status_ptr(device);
    if (!p.status) MSD_FAIL(MSD_ERR_CUDA, "fused backward: cannot locate the device status word");
    int grid = sm_count(device);
    if (p.num_tiles < grid) grid = (int)p.num_tiles;
    if (grid > kMaxGrid) grid = kMaxGrid;
    char *ws = (char *)a.ws;
    if (do_k) p.part_k = (float *)ws;
    const bool do_b = a.gb != nullptr;
    if (do_b) p.part_b = (float *)(ws + (((size_t)grid * C * taps * sizeof(float) + 255) & ~(size_t)255));
    const int mode = do_x && do_k ? 2 : (do_k ? 1 : 0);
    BwdLaunchFn fn = a.nd == 3 ? bwd3d_launchers[pl.txq16][mode] : bwd2d_launchers[pl.txq16][pl.j - 1][mode];
    int rc = fn(p, grid, pl.smem, s);
    if (rc) return rc;
    count_launch(true);
    if (do_k) {
        if ((rc = generic::reduce_partials_f32(p.part_k, grid, C * taps, C * taps, a.gk, s))) return rc;
    }
    if (do_b) {
        if ((rc = generic::reduce_partials_f32(p.part_b, grid, 1, 1, a.gb, s))) return rc;
    }
    return MSD_OK;
}

}  // namespace fast
}  // namespace msd

// Launch-variant table of the tuned kernels: which tile shape each (kernel family,
// dilation) uses.  The Python autotuner times the variants on the caller's shapes and
// records the winners here through msd_tuning_set().
#include <mutex>
#include "kernels.h"
#include "tma.cuh"

namespace msd {
namespace fast {

static const int kMaxDilation = 32;
static int g_choice[NUM_FAMILIES][kMaxDilation + 1];
static std::once_flag g_once;
static std::mutex g_mu;

static void init_table() {
    for (int f = 0; f < NUM_FAMILIES; ++f)
        for (int d = 0; d <= kMaxDilation; ++d) g_choice[f][d] = -1;
}

int tuning_set(int family, int dilation, int variant) {
    std::call_once(g_once, init_table);
    if (family < 0 || family >= NUM_FAMILIES || dilation < 0 || dilation > kMaxDilation) return MSD_ERR_BAD_ARGUMENT;
    if (variant < -1 || variant >= num_variants(family)) return MSD_ERR_BAD_ARGUMENT;
    std::lock_guard<std::mutex> l(g_mu);
    g_choice[family][dilation] = variant;
    return MSD_OK;
}

int tuning_get(int family, int dilation) {
    std::call_once(g_once, init_table);
    if (family < 0 || family >= NUM_FAMILIES || dilation < 0 || dilation > kMaxDilation) return -1;
    std::lock_guard<std::mutex> l(g_mu);
    return g_choice[family][dilation];
}

static thread_local int t_z0 = 0, t_z1 = 0;

void set_z_window(int z0, int z1) { t_z0 = z0, t_z1 = z1; }

static thread_local int t_phase = FWD_BOTH;
void set_forward_phase(int phase) { t_phase = phase; }
int get_forward_phase() { return t_phase; }

void get_z_window(int Z, int *z0, int *zw) {
    if (t_z1 > t_z0 && t_z0 >= 0 && t_z1 <= Z) {
        *z0 = t_z0;
        *zw = t_z1 - t_z0;
    } else {
        *z0 = 0;
        *zw = Z;
    }
}

}  // namespace fast

namespace tma {
static thread_local bool t_overlap = false;
bool overlap_allowed() { return t_overlap; }
void set_overlap_allowed(bool on) { t_overlap = on; }
}  // namespace tma
}  // namespace msd

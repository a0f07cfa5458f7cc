// Shared host/device helpers of the msd_b200 library.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include "../../include/msd_b200.h"

namespace msd {

// ---- error reporting (thread-local message, status codes from msd_b200.h) ----
void set_error(const char *fmt, ...);
extern thread_local char g_error[512];

#define MSD_FAIL(code, ...)            \
    do {                               \
        ::msd::set_error(__VA_ARGS__); \
        return (code);                 \
    } while (0)

#define MSD_CUDA_TRY(expr)                                                                     \
    do {                                                                                       \
        cudaError_t e__ = (expr);                                                              \
        if (e__ != cudaSuccess) {                                                              \
            ::msd::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, \
                             __LINE__);                                                        \
            return MSD_ERR_CUDA;                                                               \
        }                                                                                      \
    } while (0)

// Switches to `device` for the lifetime of the object.
struct DeviceGuard {
    int prev = -1;
    bool changed = false;
    cudaError_t status = cudaSuccess;
    explicit DeviceGuard(int device) {
        status = cudaGetDevice(&prev);
        if (status == cudaSuccess && prev != device) {
            status = cudaSetDevice(device);
            changed = (status == cudaSuccess);
        }
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(prev);
    }
};

void count_launch(bool fast);
void count_split_launch();
void count_mma_launch();    // launches of the tensor-core 3D backward kernel (likewise)  // launches of the role-split 3D backward kernel (a subset of the tuned launches)

// ---- kernel-side tensor view: N, C, then up to three spatial axes (Z, Y, X) ----
// 2D tensors are stored with a unit Z axis so that one set of kernels serves both.
struct View {
    void *p;
    int64_t n, c, z, y, x;       // sizes
    int64_t sn, sc, sz, sy, sx;  // strides in elements
};

inline bool make_view(const msd_tensor_t *t, View *v) {
    if (!t || !t->data || (t->ndim != 4 && t->ndim != 5)) return false;
    v->p = t->data;
    v->n = t->size[0];
    v->c = t->size[1];
    v->sn = t->stride[0];
    v->sc = t->stride[1];
    if (t->ndim == 4) {
        v->z = 1;
        v->sz = 0;
        v->y = t->size[2];
        v->x = t->size[3];
        v->sy = t->stride[2];
        v->sx = t->stride[3];
    } else {
        v->z = t->size[2];
        v->y = t->size[3];
        v->x = t->size[4];
        v->sz = t->stride[2];
        v->sy = t->stride[3];
        v->sx = t->stride[4];
    }
    return true;
}

// Edge-inclusive reflection: -k -> k-1, n-1+k -> n-k (one fold; needs |overshoot| <= n).
__host__ __device__ __forceinline__ int reflect(int i, int n) {
    if (i < 0) return -i - 1;
    if (i >= n) return 2 * n - i - 1;
    return i;
}

static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace msd

// Thin inline-PTX wrappers for the sm_100a tensor-core path (tcgen05): tensor-memory
// allocation, shared-memory matrix descriptors, the TF32 MMA with its accumulator in tensor
// memory, commit-to-mbarrier, and tensor-memory loads.  Single-CTA forms only
// (cta_group::1); no cluster multicast is used anywhere.
#pragma once
#include <stdint.h>
#include "tma.cuh"

namespace msd {
namespace umma {

// ---- tensor memory (TMEM): 128 lanes x 512 columns of 32 bits per SM ----
// One full warp allocates `ncols` (a power of two >= 32) columns and writes the base address
// (lane 0, first column) to `smem_dst`; the same warp frees them before the kernel ends.
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tma::smem_u32(smem_dst)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Orders tcgen05 operations of this thread with respect to barriers / other threads.
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- shared-memory matrix descriptor, 128-byte swizzle ----
// The operand tile consists of 1024-byte atoms: 8 rows of 128 bytes whose 16-byte chunks are
// XOR-permuted by the row index (chunk ^= row & 7; what TMA's 128-byte swizzle writes).
//   K-major operand  (rows = M or N index, 128 contiguous bytes = 32 consecutive k):
//       atoms of 8 rows follow each other at `sbo` bytes; `lbo` is not used.  One MMA
//       consumes 8 k (32 bytes): advance the start address by 32 bytes per k-step.
//   MN-major operand (rows = k index, 128 contiguous bytes = 32 consecutive m or n):
//       one MMA consumes one atom (8 k) per 32 m; blocks of 32 m follow at `lbo` bytes,
//       the next 8 k at `sbo` bytes.
// Bases must be 1024-byte aligned (plus the 32-byte k advance inside an atom).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);        // bits  0..13: start address / 16
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;  // bits 16..29: leading-dimension byte offset / 16
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;  // bits 32..45: stride-dimension byte offset / 16
    d |= (uint64_t)1 << 46;                           // bits 46..47: descriptor version of sm_100
    d |= (uint64_t)2 << 61;                           // bits 61..63: 128-byte swizzle
    return d;
}

// ---- instruction descriptor of kind::tf32 with float32 accumulation ----
// bits 4..5 accumulator format (1 = F32), 7..9 / 10..12 A / B format (2 = TF32), bit 15 / 16
// A / B is MN-major, 17..22 N / 8, 24..28 M / 16.
__host__ __device__ constexpr uint32_t idesc_tf32(int m, int n, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.  `accumulate` = 0 overwrites D.
__device__ __forceinline__ void mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrives (count 1) on `bar` once every MMA issued so far by this thread has completed;
// implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tma::smem_u32(bar)) : "memory");
}

// Loads 16 consecutive columns of the calling warp's 32 lanes (lane of the TMEM address =
// 32 * (warp id % 4)): thread i of the warp receives lane 32 * (warp % 4) + i.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// The same in two steps, so that a load can be in flight while the previous one's values are
// used: `v` must not be read before tmem_ld_wait().
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]),
          "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Byte offset of element (row, col) of a [rows][32 floats] tile stored as 128-byte-swizzled
// rows (rows grouped by 8 into 1024-byte atoms that follow each other densely).
__device__ __forceinline__ uint32_t sw128_offset(int row, int col) {
    return (uint32_t)(row * 128 + ((((col >> 2) ^ (row & 7)) << 4) | ((col & 3) << 2)));
}

// The value the tensor core uses for a float32 operand of kind::tf32 keeps 10 mantissa bits.
// Splitting x = hi + lo with hi exactly representable (low 13 bits cleared) and feeding
// hi*hi' + lo*hi' + hi*lo' into a float32 accumulator restores float32-level accuracy
// ("3xTF32"); lo itself has at most 13 significant bits, of which the hardware keeps 11.
__device__ __forceinline__ float tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

}  // namespace umma
}  // namespace msd

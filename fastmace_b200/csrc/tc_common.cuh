// tcgen05 / TMEM / mbarrier / bulk-copy primitives for sm_100a shared by the kernels that drive the tensor cores
// themselves (inline PTX; there is no library underneath).
#pragma once

#include "fmb_common.cuh"

namespace fmb {
namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major operand tiles with the 128-byte swizzle: a [rows][64] fp32 tile is two K halves of [rows][32] (128-byte
// rows, 1024-byte groups of 8 rows); inside a row the 16-byte chunk index is XORed with (row mod 8).
template <int ROWS>
__device__ __forceinline__ uint32_t tile_offset(int row, int k) {
    const int half = k >> 5, chunk = (k >> 2) & 7;
    return (uint32_t)(half * (ROWS * 128) + (row >> 3) * 1024 + (row & 7) * 128 + ((chunk ^ (row & 7)) << 4) + (k & 3) * 4);
}

// shared-memory matrix descriptor: start address (16-byte units), 1024 bytes between 8-row groups, descriptor
// version 1, 128-byte swizzle
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffff) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// descriptor increment (16-byte units) of K step k8 (8 elements = 32 bytes) inside a [ROWS][64] tile
template <int ROWS>
__device__ __forceinline__ uint64_t k_step(int k8) {
    return (uint64_t)(((k8 >> 2) * (ROWS * 128) + (k8 & 3) * 32) >> 4);
}

// instruction descriptor: D fp32, A and B tf32, both K-major, M = 128, N = TN
template <int TN>
__device__ __forceinline__ uint32_t make_idesc() {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ float tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, int accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n"
        :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// completion of every tcgen05 operation this thread issued so far arrives (once) on the mbarrier
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done != 0;
}

// Bounded wait shared by every role of a kernel: `abort` is a flag in shared memory; once any wait has given up the
// others return at once, so the kernel runs to its end (with meaningless results and the error word raised) instead of
// spinning.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort, unsigned limit) {
    if (mbar_try(bar, parity)) return true;                 // the common case costs one instruction
    for (unsigned spin = 1; spin < limit; ++spin) {
        if (mbar_try(bar, parity)) return true;
        if ((spin & 63u) == 63u && *abort) return false;
    }
    *abort = 1;
    return false;
}

// bulk copy global -> shared memory of this CTA (no multicast); completion counts bytes on the mbarrier
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(slot), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(base), "r"(columns) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// four consecutive accumulator columns of this thread's lane; the wait is part of the same statement so that no use
// of the registers can be scheduled before it
__device__ __forceinline__ void tmem_load_4(uint32_t taddr, float (&v)[4]) {
    uint32_t r0, r1, r2, r3;
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=&r"(r0), "=&r"(r1), "=&r"(r2), "=&r"(r3) : "r"(taddr) : "memory");
    v[0] = __uint_as_float(r0); v[1] = __uint_as_float(r1); v[2] = __uint_as_float(r2); v[3] = __uint_as_float(r3);
}

// the same for two addresses (values and their d/dr) with one wait
__device__ __forceinline__ void tmem_load_4x2(uint32_t taddr_a, uint32_t taddr_b, float (&a)[4], float (&b)[4]) {
    uint32_t r0, r1, r2, r3, q0, q1, q2, q3;
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%8];\n"
        "tcgen05.ld.sync.aligned.32x32b.x4.b32 {%4, %5, %6, %7}, [%9];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=&r"(r0), "=&r"(r1), "=&r"(r2), "=&r"(r3), "=&r"(q0), "=&r"(q1), "=&r"(q2), "=&r"(q3)
        : "r"(taddr_a), "r"(taddr_b) : "memory");
    a[0] = __uint_as_float(r0); a[1] = __uint_as_float(r1); a[2] = __uint_as_float(r2); a[3] = __uint_as_float(r3);
    b[0] = __uint_as_float(q0); b[1] = __uint_as_float(q1); b[2] = __uint_as_float(q2); b[3] = __uint_as_float(q3);
}

// N consecutive accumulator columns of this thread's lane (N = 8 or 16), wait included
__device__ __forceinline__ void tmem_load_8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]), "=&r"(r[7])
        : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]), "=&r"(r[7]),
          "=&r"(r[8]), "=&r"(r[9]), "=&r"(r[10]), "=&r"(r[11]), "=&r"(r[12]), "=&r"(r[13]), "=&r"(r[14]), "=&r"(r[15])
        : "r"(taddr) : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// two groups of 16 columns with one wait
__device__ __forceinline__ void tmem_load_16x2(uint32_t taddr_a, uint32_t taddr_b, float (&a)[16], float (&b)[16]) {
    uint32_t r[16], q[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%32];\n"
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%33];\n"
        "tcgen05.wait::ld.sync.aligned;"
        : "=&r"(r[0]), "=&r"(r[1]), "=&r"(r[2]), "=&r"(r[3]), "=&r"(r[4]), "=&r"(r[5]), "=&r"(r[6]), "=&r"(r[7]),
          "=&r"(r[8]), "=&r"(r[9]), "=&r"(r[10]), "=&r"(r[11]), "=&r"(r[12]), "=&r"(r[13]), "=&r"(r[14]), "=&r"(r[15]),
          "=&r"(q[0]), "=&r"(q[1]), "=&r"(q[2]), "=&r"(q[3]), "=&r"(q[4]), "=&r"(q[5]), "=&r"(q[6]), "=&r"(q[7]),
          "=&r"(q[8]), "=&r"(q[9]), "=&r"(q[10]), "=&r"(q[11]), "=&r"(q[12]), "=&r"(q[13]), "=&r"(q[14]), "=&r"(q[15])
        : "r"(taddr_a), "r"(taddr_b) : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) { a[i] = __uint_as_float(r[i]); b[i] = __uint_as_float(q[i]); }
}

template <int N> __device__ __forceinline__ void tmem_load(uint32_t taddr, float (&v)[N]) {
    static_assert(N == 4 || N == 8 || N == 16, "tmem_load: 4, 8 or 16 columns");
    if constexpr (N == 4) tmem_load_4(taddr, v);
    else if constexpr (N == 8) tmem_load_8(taddr, v);
    else tmem_load_16(taddr, v);
}

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}

}  // namespace tc
}  // namespace fmb

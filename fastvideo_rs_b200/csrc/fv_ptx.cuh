// Thin inline-PTX layer for the sm_100a attention kernels: mbarrier (with
// bounded waits), TMA tiled loads, tcgen05 MMA / commit / TMEM load-store.
//
// Every wait in this file is bounded.  A wait that outlives FV_WAIT_CYCLES
// records a code in the global status word, raises the CTA's abort flag and
// returns false; the caller then leaves its role loop and falls through to the
// common kernel exit (drain copies in flight, free TMEM, return).  No trap, no
// endless spin: the context stays usable and the host reads the status word.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define FV_DEV __device__ __forceinline__

// ~0.25 s at 2 GHz.  A healthy wait on this path is microseconds.
#ifndef FV_WAIT_CYCLES
#define FV_WAIT_CYCLES 500000000ll
#endif

// Status word codes (device -> host).
#define FV_ST_OK 0
#define FV_ST_TIMEOUT_BASE 100  // + role id

namespace fvp {

FV_DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ------------------------------------------------------------------ mbarrier
FV_DEV void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
FV_DEV void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
FV_DEV void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
FV_DEV void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
FV_DEV uint32_t mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// try_wait with an explicit limit (nanoseconds) on how long the thread may stay suspended before it looks again.
FV_DEV uint32_t mbar_try_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok;
}

// Non-blocking probe of phase `parity` (test_wait never suspends the thread).
FV_DEV uint32_t mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok;
}

// What a role needs to give up cleanly: the CTA's abort flag (shared) and the
// launch's status word (global).
struct WaitCtl {
    volatile int* abort_smem;
    int* status;
    int role;
    long long limit = FV_WAIT_CYCLES;  // cycles a wait may last before the role gives up
};

// Bounded wait on phase `parity`.  Returns false after a timeout or when
// another thread of the CTA (or an earlier CTA of the launch) already gave up.
FV_DEV bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtl& c) {
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    uint32_t n = 0;
    while (!mbar_try(bar, parity)) {
        if (((++n) & 63u) == 0u) {
            if (*c.abort_smem) return false;
            if (clock64() - t0 > c.limit) {
                *c.abort_smem = 1;
                atomicCAS(c.status, FV_ST_OK, FV_ST_TIMEOUT_BASE + c.role);
                return false;
            }
        }
    }
    return true;
}

// ----------------------------------------------------------------------- TMA
FV_DEV void tma_prefetch_desc(const void* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// 4-D tiled load (coordinates innermost first), completion on an mbarrier.
FV_DEV void tma_load4(uint32_t dst, const void* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// 1-D bulk copy global -> shared, completion on an mbarrier.  Both addresses and the size are multiples of 16 bytes.
FV_DEV void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
// Bounded wait that ignores the abort flag: the exit path uses it to let copies in flight land.
FV_DEV bool mbar_drain(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    while (!mbar_try(bar, parity)) {
        if (clock64() - t0 > FV_WAIT_CYCLES) return false;
    }
    return true;
}

FV_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
FV_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

FV_DEV void tmem_alloc(uint32_t slot_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
FV_DEV void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle:
// bits 0-13 start>>4, 16-29 leading byte offset>>4, 32-45 stride byte
// offset>>4, bit 46 descriptor version (1 on sm_100), bits 61-63 swizzle
// mode (2 = 128 B).  K-major operand: 8-row groups are `sbo` apart (1024 B for
// 128-byte rows) and `lbo` is ignored.  MN-major operand: 64-element chunks
// along MN are `lbo` apart, 8-row groups along K are `sbo` apart.
FV_DEV uint64_t umma_desc_sw128(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor for kind::f16: f32 accumulator (bits 4-5 = 1), bf16
// A and B (bits 7-9 = 1, 10-12 = 1), A K-major (bit 15 = 0), B major at bit
// 16 (0 = K-major, 1 = MN-major), N>>3 at bits 17-22, M>>4 at bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(uint32_t M, uint32_t N, uint32_t b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn_major << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]
FV_DEV void umma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
FV_DEV void umma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d), "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One arrival on `bar` when every tcgen05 op issued so far by this thread is done.
FV_DEV void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

#define FV_O4(r, i) "=r"(r[i]), "=r"(r[i + 1]), "=r"(r[i + 2]), "=r"(r[i + 3])
#define FV_O16(r, i) FV_O4(r, i), FV_O4(r, i + 4), FV_O4(r, i + 8), FV_O4(r, i + 12)
#define FV_O32(r, i) FV_O16(r, i), FV_O16(r, i + 16)
#define FV_I4(r, i) "r"(r[i]), "r"(r[i + 1]), "r"(r[i + 2]), "r"(r[i + 3])
#define FV_I16(r, i) FV_I4(r, i), FV_I4(r, i + 4), FV_I4(r, i + 8), FV_I4(r, i + 12)
#define FV_I32(r, i) FV_I16(r, i), FV_I16(r, i + 16)
#define FV_L32_A "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}"
#define FV_L32_B "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32}"

// Issue a load of 32 consecutive 32-bit TMEM columns of this thread's lane
// (warp w of a warpgroup may touch lanes 32*(w%4)..+31 only).  The registers
// are NOT valid until tmem_ld_wait() followed by tmem_pin32() on them.
template <int OFF>
FV_DEV void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[128]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 " FV_L32_A ", [%32];" : FV_O32(r, OFF) : "r"(taddr) : "memory");
}
FV_DEV void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 " FV_L32_A ", [%32];" : FV_O32(r, 0) : "r"(taddr) : "memory");
}
// The same for register arrays of other sizes: 32 columns into r[OFF .. OFF+31].
template <int OFF, int N>
FV_DEV void tmem_ld32_at(uint32_t taddr, uint32_t (&r)[N]) {
    static_assert(OFF + 32 <= N, "tmem_ld32_at: out of range");
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 " FV_L32_A ", [%32];" : FV_O32(r, OFF) : "r"(taddr) : "memory");
}
FV_DEV void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
FV_DEV void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Orders every later use of r after the preceding volatile asm (the wait):
// volatile asm statements keep their program order, and the consumers of r
// now depend on this one.
template <int N>
FV_DEV void tmem_pin(uint32_t (&r)[N]) {
#pragma unroll
    for (int i = 0; i < N; i++) asm volatile("" : "+r"(r[i]));
}
// Store 32 registers to 32 consecutive TMEM columns of this thread's lane.
FV_DEV void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], " FV_L32_B ";" ::"r"(taddr), FV_I32(r, 0) : "memory");
}

// Store r[OFF .. OFF+31] to 32 consecutive TMEM columns of this thread's lane.
template <int OFF, int N>
FV_DEV void tmem_st32_at(uint32_t taddr, const uint32_t (&r)[N]) {
    static_assert(OFF + 32 <= N, "tmem_st32_at: out of range");
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], " FV_L32_B ";" ::"r"(taddr), FV_I32(r, OFF) : "memory");
}
// Store 16 registers to 16 consecutive TMEM columns of this thread's lane.
FV_DEV void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    constexpr int OFF = 0;
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), FV_I16(r, OFF)
        : "memory");
}

// Store r[OFF .. OFF+15] to 16 consecutive TMEM columns of this thread's lane.
template <int OFF, int N>
FV_DEV void tmem_st16_at(uint32_t taddr, const uint32_t (&r)[N]) {
    static_assert(OFF + 16 <= N, "tmem_st16_at: out of range");
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), FV_I16(r, OFF)
        : "memory");
}

// --------------------------------------------------------------------- math
FV_DEV float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// bf16x2 word: `lo` in bits 0-15, `hi` in bits 16-31, round to nearest even.
FV_DEV uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Packed pairs of f32 (sm_100 has two-wide FADD / FMUL / FFMA on 64-bit register pairs).
FV_DEV uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
FV_DEV void unpack_f32x2(uint64_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
FV_DEV uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
FV_DEV uint64_t add_f32x2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
FV_DEV float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 2^x for a pair, on the FMA pipe (no MUFU): x = n + f with n = round(x), f in [-0.5, 0.5];
// 2^f by a cubic fitted to a relative error of 7.5e-5 (far inside the bf16 rounding of P, 3.9e-3);
// 2^n by adding n to the exponent field.  x is clamped to -126 (result ~1e-38, never a denormal path).
FV_DEV void ex2_poly_x2(float x0, float x1, float& p0, float& p1) {
    const float MAGIC = 12582912.f;  // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
    x0 = fmaxf(x0, -126.f);
    x1 = fmaxf(x1, -126.f);
    const uint64_t x = pack_f32x2(x0, x1);
    const uint64_t r = add_f32x2(x, pack_f32x2(MAGIC, MAGIC));
    float r0, r1;
    unpack_f32x2(r, r0, r1);
    const uint64_t rn = add_f32x2(r, pack_f32x2(-MAGIC, -MAGIC));
    // f = x - round(x)
    const uint64_t f = fma_f32x2(rn, pack_f32x2(-1.f, -1.f), x);
    uint64_t p = fma_f32x2(f, pack_f32x2(0.055171408f, 0.055171408f), pack_f32x2(0.24261075f, 0.24261075f));
    p = fma_f32x2(p, f, pack_f32x2(0.69326097f, 0.69326097f));
    p = fma_f32x2(p, f, pack_f32x2(0.9999281f, 0.9999281f));
    float q0, q1;
    unpack_f32x2(p, q0, q1);
    p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(r0) << 23));
    p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(r1) << 23));
}

}  // namespace fvp

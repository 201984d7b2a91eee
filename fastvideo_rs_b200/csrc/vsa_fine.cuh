// The fine stage of Video Sparse Attention on sm_100a: softmax(q k^T scale) v of every query tile (64 tokens of
// a 4 x 4 x 4 cube) over the key tiles its row of `selected` names, with Wan's combine
// out[token] = coarse[tile] * gate[token] + fine and the scatter from slot order to token order in the epilogue.
//
// Replaces the launcher attn_dc::vsa_fine and the kernel it loads (crates/fastvideo-cudarc/src/rt/attn_dc.rs:387-506,
// rt/attn_dc.cu:790-1257) plus the separate combine launch (rt/ops.rs:1554-1619), behind vsa_attention_device
// (rt/vsa.rs:358-470).
//
// Shape of the kernel (the roles and hand-overs are those of attn_fwd.cuh, cut to a 64-key step)
// -----------------------------------------------------------------------------------------------
// * One CTA per PAIR of query tiles (M = 128 rows: tile 2p in rows 0-63, tile 2p+1 in rows 64-127) and plane;
//   256 TMEM columns (two score buffers of 64 columns, one accumulator of 128) and about 100 KB of shared
//   memory, so two CTAs share an SM and one's softmax runs under the other's products.
// * The pair walks the ASCENDING UNION of its two selections, one 64-key tile per step.  A list entry carries
//   the key tile, its number of real keys and which of the two query tiles selected it; the rows of the
//   other one store P = 0 for that step and skip the exponentials.
// * 6 warps: 0-3 softmax (thread = TMEM lane = row), 4 builds the union and then loads (one thread), 5
//   issues the products (one thread) and owns the TMEM allocation.
// * Q.K^T runs two steps ahead of P.V (score buffers alternate), so the softmax of step j + 1 starts when
//   that of step j ends.  K/V arrive in UNITS [V(j) | K(j+2)]: what step j's P.V and the Q.K^T issued right
//   after it read, one "full" and one "free" barrier per unit -- per step the issuer passes two waits
//   (the unit, P) and four commits.
// * Softmax without a maximum pass, as in the dense kernel: P = 2^(s sl2 - m) against the row's lazy
//   reference, the row sum as the guard, and an out-of-line exact path for the first visible tile of a row,
//   ragged tiles (fewer than 64 real keys) and tripped guards.  The exact path may rescale O, which the
//   product of the step before may still be updating: it waits for that product (pv_done) first.
// * Every wait is bounded (WaitCtl: abort flag + status word); all roles leave through the common exit.
#pragma once
#include <cuda.h>
#include "attn_fwd.cuh"

namespace fvvsa {

using namespace fvp;

constexpr int kFineThreads = 192;
constexpr int kUnits = 2;                   // units of the K/V ring
constexpr uint32_t kKeyTileB = 16384;       // 64 keys x 128 bf16: two 8 KB panels
constexpr uint32_t kKeyPanelB = 8192;
constexpr uint32_t kUnitB = 2 * kKeyTileB;  // [V | K]
constexpr uint32_t kQPairB = 32768;         // 128 rows x 128 bf16: two 16 KB panels
constexpr uint32_t kQPanelB = 16384;
constexpr int kTileSlots = 64;              // slots of a 4 x 4 x 4 tile

// Offsets from the 1024-byte aligned start of dynamic shared memory.
struct FineSmem {
    static constexpr uint32_t q = 0;
    static constexpr uint32_t ring = q + kQPairB;
    static constexpr uint32_t q_full = ring + kUnits * kUnitB;   // barriers, 8 bytes each
    static constexpr uint32_t unit_full = q_full + 8;            // [kUnits]
    static constexpr uint32_t unit_free = unit_full + 8 * kUnits;
    static constexpr uint32_t s_ready = unit_free + 8 * kUnits;  // [2] score buffer written (issuer -> softmax)
    static constexpr uint32_t p_ready = s_ready + 16;            // [2] P stored there by the four softmax warps
    static constexpr uint32_t pv_done = p_ready + 16;            // one phase per P.V (issuer -> exact softmax path)
    static constexpr uint32_t o_ready = pv_done + 8;             // the last P.V
    static constexpr uint32_t drain = o_ready + 8;
    static constexpr uint32_t tmem_slot = drain + 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t count = abort_flag + 4;            // entries of the union
    static constexpr uint32_t list = q_full + 256;               // the union, then two staging areas of topk words
    static constexpr size_t bytes(int list_cap, int topk) { return 1024 + (size_t)list + 4 * ((size_t)list_cap + 2 * (size_t)topk); }
};
static_assert(FineSmem::count + 4 <= FineSmem::list, "barrier block overlaps the list");

struct FineJob {
    const uint32_t* selected;     // [planes, tiles, topk] ascending
    const uint32_t* block_sizes;  // [tiles] real keys of a tile
    const int32_t* slot_src;      // [tiles * 64] token of a slot, -1 for padding
    const float* coarse;          // [planes, tiles, 128]
    const __nv_bfloat16* gate;    // [planes, seq, 128] or null (gate of one)
    void* out;                    // [planes, seq, 128]
    int* status;
    int out_is_bf16;
    int planes, tiles, topk, seq;
    float sl2;
    int list_cap;
};

// A union entry: key tile (20 bits) | real keys (7 bits at 20) | selected by query tile 0 / 1 (bits 27, 28).
FV_DEV uint32_t entry_tile(uint32_t e) { return e & 0xFFFFFu; }
FV_DEV int entry_keys(uint32_t e) { return (int)((e >> 20) & 127u); }
FV_DEV bool entry_for(uint32_t e, int which) { return ((e >> (27 + which)) & 1u) != 0u; }

#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL) || !defined(__CUDA_ARCH__)

// The union of two ascending selections by one warp: both lists staged in shared memory, one lane merges, every
// lane then adds the real-key counts.
FV_DEV int build_union(const FineJob& jb, int plane, int qt0, int qt1, volatile uint32_t* list, int lane) {
    const uint32_t* la = jb.selected + ((size_t)plane * jb.tiles + qt0) * jb.topk;
    const uint32_t* lb = jb.selected + ((size_t)plane * jb.tiles + qt1) * jb.topk;
    const int na = jb.topk, nb = qt1 < jb.tiles ? jb.topk : 0;
    volatile uint32_t* sa = list + jb.list_cap;
    volatile uint32_t* sb = sa + jb.topk;
    for (int i = lane; i < na; i += 32) sa[i] = la[i];
    for (int i = lane; i < nb; i += 32) sb[i] = lb[i];
    __syncwarp();
    int n = 0;
    if (lane == 0) {
        int i = 0, j = 0;
        while ((i < na || j < nb) && n < jb.list_cap) {
            const uint32_t a = i < na ? sa[i] : 0xffffffffu, b = j < nb ? sb[j] : 0xffffffffu;
            if (a < b) list[n++] = a | (1u << 27), i++;
            else if (b < a) list[n++] = b | (2u << 27), j++;
            else list[n++] = a | (3u << 27), i++, j++;
        }
    }
    n = __shfl_sync(0xffffffffu, n, 0);
    __syncwarp();
    for (int i = lane; i < n; i += 32) {
        const uint32_t e = list[i];
        list[i] = e | (min(jb.block_sizes[entry_tile(e)], (uint32_t)kTileSlots) << 20);
    }
    return n;
}

// S (128 rows x 64 keys, f32) = Q (128 x 128, K-major, SW128) . K^T (64 keys x 128): eight K = 16 slices; inside a
// panel a slice is 32 bytes (2 address units) on, the second panel 16 KB (Q) or 8 KB (K) on.
FV_DEV void scores64_mma(uint32_t tS, uint64_t qd, uint64_t kd) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, 64, 0);
#define FV_QK64(oa, ob) "add.s64 a, %1, " #oa ";\n\tadd.s64 b, %2, " #ob ";\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
    asm volatile(
        "{\n\t.reg .pred pt, pf;\n\t.reg .b64 a, b;\n\t"
        "setp.ne.b32 pf, %3, %3;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
        FV_QK64(2, 2) FV_QK64(4, 4) FV_QK64(6, 6) FV_QK64(1024, 512) FV_QK64(1026, 514) FV_QK64(1028, 516) FV_QK64(1030, 518)
        "}"
        ::"r"(tS), "l"(qd), "l"(kd), "r"(idesc)
        : "memory");
#undef FV_QK64
}
// O (128 x 128 f32) (+)= P (TMEM, 64 keys as 32 bf16x2 columns) . V (64 keys x 128, MN-major): four K = 16 slices,
// 8 columns of P and 2 KB of V each.
FV_DEV void output64_mma(uint32_t tO, uint32_t tP, uint64_t vd, bool accumulate) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, 128, 1);
#define FV_PV64(col, off) "add.u32 t, %1, " #col ";\n\tadd.s64 b, %2, " #off ";\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
    asm volatile(
        "{\n\t.reg .pred pt, p0;\n\t.reg .b64 b;\n\t.reg .b32 t;\n\t"
        "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
        FV_PV64(8, 128) FV_PV64(16, 256) FV_PV64(24, 384)
        "}"
        ::"r"(tO), "r"(tP), "l"(vd), "r"(idesc), "r"(accumulate ? 1u : 0u)
        : "memory");
#undef FV_PV64
}

struct FineRow {
    float m, l;  // lazy reference (base 2, -inf = none yet) and the sum of P against it
};

// The exact way through one 64-key step for rows that see the tile: padding keys hidden, exact row maximum,
// reference moved where it is missing or more than 2^8 behind (O and the row sum follow), MUFU exponentials.
// O may still be under the product of the step before: that product is awaited before O is touched.
static __device__ __noinline__ bool fine_careful(uint32_t tS, uint32_t tO, uint32_t sbase, int step, int keys, float sl2, int lane,
                                          const WaitCtl& ctl, FineRow* rs) {
    using namespace fvattn;
    float m = rs->m, l = rs->l;
    uint32_t u0[32], u1[32];
    load_chunk(tS, 0, u0);
    load_chunk(tS, 1, u1);
    land_chunk(u0);
    tmem_pin(u1);
    if (keys < kTileSlots) {
#pragma unroll
        for (int c = 0; c < 32; c++) {
            u0[c] = c < keys ? u0[c] : as_u(neg_inf());
            u1[c] = 32 + c < keys ? u1[c] : as_u(neg_inf());
        }
    }
    const float cand = fmaxf(max32(u0), max32(u1)) * sl2;
    float a = 1.f;
    if (cand > m + 8.f) {
        a = ex2(m - cand);  // 0 when there was no reference
        m = cand;
        l *= a;
    }
    if (step > 0 && __any_sync(kFullWarp, a != 1.f)) {
        if (!__all_sync(kFullWarp, mbar_wait(sbase + FineSmem::pv_done, (uint32_t)(step - 1) & 1u, ctl))) return false;
        tc_fence_after();
#pragma unroll 1
        for (int q = 0; q < 4; q++) {
            uint32_t o[32];
            tmem_ld32_issue(tO + 32u * q, o);
            tmem_ld_wait();
            tmem_pin(o);
#pragma unroll
            for (int c = 0; c < 32; c++) o[c] = as_u(as_f(o[c]) * a);
            tmem_st32(tO + 32u * q, o);
        }
    }
    const float noff = (m == neg_inf()) ? 0.f : -m;
    const uint64_t s2 = pack_f32x2(sl2, sl2), nf = pack_f32x2(noff, noff);
    uint32_t pw[32];
    uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
    float top = 0.f;
    exp32<false>(u0, pw, s2, nf, acc0, acc1, top);
    exp32<false>(u1, pw + 16, s2, nf, acc0, acc1, top);
    l += part_sum<false>(acc0, acc1, top);
    tmem_st32(tS, pw);
    rs->m = m;
    rs->l = l;
    return true;
}

// ------------------------------------------------------------------------------------------ softmax warps
FV_DEV void fine_softmax(const FineJob& jb, uint32_t sbase, uint32_t tmem, volatile const uint32_t* list, int nent, int plane,
                         int qt0, int qt1, int warp, int lane, const WaitCtl& ctl) {
    using namespace fvattn;
    const int row = warp * 32 + lane, which = row >> 6;  // rows 0-63: query tile qt0, rows 64-127: qt1 (a warp lies in one)
    const uint32_t lanes = tmem + ((uint32_t)(warp * 32) << 16);
    const uint32_t tO = lanes + 128u;
    const float sl2 = jb.sl2;
    FineRow rs{neg_inf(), 0.f};
    bool ok = true;
#pragma unroll 1
    for (int j = 0; j < nent; j++) {
        const uint32_t e = list[j];
        const int keys = entry_keys(e);
        const uint32_t buf = (uint32_t)j & 1u, tS = lanes + 64u * buf;
        if (!__all_sync(kFullWarp, mbar_wait(sbase + FineSmem::s_ready + 8u * buf, (uint32_t)(j >> 1) & 1u, ctl))) { ok = false; break; }
        tc_fence_after();
        if (!entry_for(e, which)) {  // (warp-uniform) not this query tile's key tile: no weight
            uint32_t z[32];
#pragma unroll
            for (int c = 0; c < 32; c++) z[c] = 0u;
            tmem_st32(tS, z);
        } else {
            bool hot = keys == kTileSlots && __all_sync(kFullWarp, rs.m != neg_inf());
            if (hot) {
                uint32_t u0[32], u1[32], pw[32];
                const uint64_t s2 = pack_f32x2(sl2, sl2), nf = pack_f32x2(-rs.m, -rs.m);
                uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
                float top = 0.f;
                load_chunk(tS, 0, u0);
                land_chunk(u0);
                load_chunk(tS, 1, u1);  // on its way under the first chunk's exponentials
                exp32<true>(u0, pw, s2, nf, acc0, acc1, top);
                land_chunk(u1);
                exp32<true>(u1, pw + 16, s2, nf, acc0, acc1, top);
                const float sum = part_sum<true>(acc0, acc1, top);
                if (__any_sync(kFullWarp, !(sum <= kGuard))) {
                    hot = false;  // nothing stored yet: the exact way
                } else {
                    tmem_st32(tS, pw);
                    rs.l += sum;
                }
            }
            if (!hot && !fine_careful(tS, tO, sbase, j, keys, sl2, lane, ctl, &rs)) { ok = false; break; }
        }
        publish(sbase + FineSmem::p_ready + 8u * buf, lane);
    }
    if (ok && nent > 0) ok = __all_sync(kFullWarp, mbar_wait(sbase + FineSmem::o_ready, 0, ctl));
    tc_fence_after();
    if (!ok) return;

    // ---- epilogue: fine / l + coarse * gate, slot order -> token order
    const int qt = which ? qt1 : qt0;
    int token = -1;
    if (qt < jb.tiles) token = jb.slot_src[qt * kTileSlots + (row & 63)];
    const bool live = token >= 0;
    const float inv = rs.l > 0.f ? 1.f / rs.l : 0.f;
    const size_t orow = ((size_t)plane * jb.seq + (live ? token : 0)) * fvattn::kD;
    const float* co = jb.coarse + ((size_t)plane * jb.tiles + min(qt, jb.tiles - 1)) * fvattn::kD;
#pragma unroll 1
    for (int q = 0; q < 4; q++) {
        uint32_t o[32];
        if (nent > 0) {
            tmem_ld32_issue(tO + 32u * q, o);
            tmem_ld_wait();
            tmem_pin(o);
        } else {
#pragma unroll
            for (int c = 0; c < 32; c++) o[c] = 0u;
        }
        if (!live) continue;
        float f[32];
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const float4 cv = *reinterpret_cast<const float4*>(co + 32 * q + 4 * c);
            float g[4] = {1.f, 1.f, 1.f, 1.f};
            if (jb.gate) {
                const uint2 gw = *reinterpret_cast<const uint2*>(jb.gate + orow + 32 * q + 4 * c);
                g[0] = as_f(gw.x << 16);
                g[1] = as_f(gw.x & 0xffff0000u);
                g[2] = as_f(gw.y << 16);
                g[3] = as_f(gw.y & 0xffff0000u);
            }
            const float cvv[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
            for (int i = 0; i < 4; i++) f[4 * c + i] = __fadd_rn(__fmul_rn(cvv[i], g[i]), as_f(o[4 * c + i]) * inv);
        }
        if (jb.out_is_bf16) {
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(jb.out) + orow + 32 * q);
#pragma unroll
            for (int c = 0; c < 4; c++)
                dst[c] = make_uint4(pack_bf16x2(f[8 * c], f[8 * c + 1]), pack_bf16x2(f[8 * c + 2], f[8 * c + 3]),
                                    pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), pack_bf16x2(f[8 * c + 6], f[8 * c + 7]));
        } else {
            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(jb.out) + orow + 32 * q);
#pragma unroll
            for (int c = 0; c < 8; c++) dst[c] = make_float4(f[4 * c], f[4 * c + 1], f[4 * c + 2], f[4 * c + 3]);
        }
    }
}

// ---------------------------------------------------------------------------------------------- loader
// Unit u (u = 0 .. nent + 1) = [V(u-2) | K(u)], either half absent at the ends; unit u lives in slot u % kUnits.
FV_DEV void fine_loader(const CUtensorMap* mk, const CUtensorMap* mv, uint32_t sbase, volatile const uint32_t* list, int nent,
                        int plane, const WaitCtl& ctl) {
    tma_prefetch_desc(mk);
    tma_prefetch_desc(mv);
    int loaded = 0;
    const int units = nent > 0 ? nent + 2 : 0;
    for (int u = 0; u < units; u++) {
        const uint32_t slot = (uint32_t)u % kUnits, use = (uint32_t)u / kUnits;
        if (use > 0 && !mbar_wait(sbase + FineSmem::unit_free + 8u * slot, (use - 1u) & 1u, ctl)) break;
        const bool has_v = u >= 2, has_k = u < nent;
        const uint32_t dst = sbase + FineSmem::ring + slot * kUnitB, bar = sbase + FineSmem::unit_full + 8u * slot;
        mbar_expect_tx(bar, (has_v ? kKeyTileB : 0u) + (has_k ? kKeyTileB : 0u));
        if (has_v) {
            const int tile = (int)entry_tile(list[u - 2]);
            tma_load4(dst, mv, bar, 0, tile * kTileSlots, plane, 0);
            tma_load4(dst + kKeyPanelB, mv, bar, 64, tile * kTileSlots, plane, 0);
        }
        if (has_k) {
            const int tile = (int)entry_tile(list[u]);
            tma_load4(dst + kKeyTileB, mk, bar, 0, tile * kTileSlots, plane, 0);
            tma_load4(dst + kKeyTileB + kKeyPanelB, mk, bar, 64, tile * kTileSlots, plane, 0);
        }
        loaded = u + 1;
    }
    // copies in flight must land before the CTA's shared memory goes away
    mbar_wait(sbase + FineSmem::q_full, 0, ctl);
    for (int s = 0; s < kUnits && s < loaded; s++) {
        const int last = ((loaded - 1 - s) / kUnits) * kUnits + s;
        mbar_wait(sbase + FineSmem::unit_full + 8u * (uint32_t)s, (uint32_t)(last / kUnits) & 1u, ctl);
    }
}

// ---------------------------------------------------------------------------------------------- issuer
// In order: S(0), S(1), then per step j: wait unit j + 2 and P(j); O += P(j) . V(j); S(j + 2) = Q . K(j + 2)^T into
// the buffer P(j) has just been read from.
FV_DEV void fine_issuer(uint32_t sbase, uint32_t tmem, int nent, const WaitCtl& ctl) {
    bool ok = mbar_wait(sbase + FineSmem::q_full, 0, ctl);
    tc_fence_after();
    const uint64_t qd = umma_desc_sw128(sbase + FineSmem::q, 16, 1024);
    auto unit_addr = [&](int u) { return sbase + FineSmem::ring + ((uint32_t)u % kUnits) * kUnitB; };
    auto unit_wait = [&](int u) {
        return mbar_wait(sbase + FineSmem::unit_full + 8u * ((uint32_t)u % kUnits), ((uint32_t)u / kUnits) & 1u, ctl);
    };
    auto scores = [&](int j) {  // K(j) is the second half of unit j
        scores64_mma(tmem + 64u * ((uint32_t)j & 1u), qd, umma_desc_sw128(unit_addr(j) + kKeyTileB, 16, 1024));
        umma_commit(sbase + FineSmem::s_ready + 8u * ((uint32_t)j & 1u));
    };
    for (int u = 0; u < 2 && u < nent && ok; u++) {  // units 0 and 1 hold K(0), K(1) only
        ok = unit_wait(u);
        if (!ok) break;
        tc_fence_after();
        scores(u);
        umma_commit(sbase + FineSmem::unit_free + 8u * ((uint32_t)u % kUnits));
    }
#pragma unroll 1
    for (int j = 0; j < nent && ok; j++) {
        const int u = j + 2;
        if (!unit_wait(u)) { ok = false; break; }
        if (!mbar_wait(sbase + FineSmem::p_ready + 8u * ((uint32_t)j & 1u), (uint32_t)(j >> 1) & 1u, ctl)) { ok = false; break; }
        tc_fence_after();
        output64_mma(tmem + 128u, tmem + 64u * ((uint32_t)j & 1u), umma_desc_sw128(unit_addr(u), kKeyPanelB, 1024), j > 0);
        umma_commit(sbase + FineSmem::pv_done);
        if (j == nent - 1) umma_commit(sbase + FineSmem::o_ready);
        if (u < nent) scores(u);
        umma_commit(sbase + FineSmem::unit_free + 8u * ((uint32_t)u % kUnits));
    }
    umma_commit(sbase + FineSmem::drain);
    mbar_wait(sbase + FineSmem::drain, 0, ctl);
}

#endif  // sm_100a / host pass

__global__ void __launch_bounds__(kFineThreads, 2)
fv_vsa_fine_kernel(const __grid_constant__ CUtensorMap mq, const __grid_constant__ CUtensorMap mk,
                   const __grid_constant__ CUtensorMap mv, const __grid_constant__ FineJob jb) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL)
    extern __shared__ unsigned char fine_smem_raw[];
    const uint32_t raw = smem_u32(fine_smem_raw);
    const uint32_t sbase = (raw + 1023u) & ~1023u;
    unsigned char* smem = fine_smem_raw + (sbase - raw);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + FineSmem::tmem_slot);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + FineSmem::abort_flag);
    volatile int* count = reinterpret_cast<volatile int*>(smem + FineSmem::count);
    volatile uint32_t* list = reinterpret_cast<volatile uint32_t*>(smem + FineSmem::list);

    const int warp = (int)(threadIdx.x >> 5), lane = (int)(threadIdx.x & 31);
    const int pairs = (jb.tiles + 1) / 2;
    const int pair = (int)(blockIdx.x % (unsigned)pairs), plane = (int)(blockIdx.x / (unsigned)pairs);
    const int qt0 = 2 * pair, qt1 = 2 * pair + 1;

    if (threadIdx.x == 0) {
        mbar_init(sbase + FineSmem::q_full, 1);
        for (int s = 0; s < kUnits; s++) {
            mbar_init(sbase + FineSmem::unit_full + 8u * s, 1);
            mbar_init(sbase + FineSmem::unit_free + 8u * s, 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(sbase + FineSmem::s_ready + 8u * b, 1);
            mbar_init(sbase + FineSmem::p_ready + 8u * b, 4);  // one arrival per softmax warp
        }
        mbar_init(sbase + FineSmem::pv_done, 1);
        mbar_init(sbase + FineSmem::o_ready, 1);
        mbar_init(sbase + FineSmem::drain, 1);
        *abort_flag = (*(volatile int*)jb.status != FV_ST_OK) ? 1 : 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (*abort_flag) return;  // CTA-uniform
    if (warp == 5) tmem_alloc(sbase + FineSmem::tmem_slot, 256);
    if (warp == 4) {
        if (lane == 0) {
            tma_prefetch_desc(&mq);
            mbar_expect_tx(sbase + FineSmem::q_full, kQPairB);
            tma_load4(sbase + FineSmem::q, &mq, sbase + FineSmem::q_full, 0, qt0 * kTileSlots, plane, 0);
            tma_load4(sbase + FineSmem::q + kQPanelB, &mq, sbase + FineSmem::q_full, 64, qt0 * kTileSlots, plane, 0);
        }
        const int n = build_union(jb, plane, qt0, qt1, list, lane);
        if (lane == 0) *count = n;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const int nent = *count;

    if (warp < 4) {
        const WaitCtl ctl{abort_flag, jb.status, 13};
        fine_softmax(jb, sbase, tmem, list, nent, plane, qt0, qt1, warp, lane, ctl);
    } else if (lane == 0) {
        if (warp == 4) fine_loader(&mk, &mv, sbase, list, nent, plane, WaitCtl{abort_flag, jb.status, 11});
        else fine_issuer(sbase, tmem, nent, WaitCtl{abort_flag, jb.status, 12});
    }
    // every TMEM access of every thread is complete: the allocation may go
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc(tmem, 256);
    }
#endif
}

}  // namespace fvvsa

// Flash-style SDPA forward for head dim 128 on sm_100a: TMA-staged Q/K/V,
// tcgen05.mma (cta_group::1, kind::f16) with TMEM accumulators, one query row
// per softmax thread.  One kernel body serves dense self/cross attention, the
// Wan block-causal mask, sequence-parallel K/V (several gathered segments) and
// the second pass of a two-pass (local keys, then remote keys) evaluation.
//
// Replaces, behind the same operand convention (bf16 [bh, s, 128] in, bf16 or
// f32 [bh, sq, 128] out, sl2 = scale * log2 e), the reference launcher
// crates/fastvideo-cudarc/src/rt/attn_dc.rs:213-273 (dense_fwd) and the
// block-causal launcher crates/fastvideo-cudarc/src/rt/attn.rs:647-730.
//
// CTA = 256 query rows of one head = two M=128 query tiles; 12 warps:
//   warps 0-3 / 4-7  softmax of query tile 0 / 1 (thread = TMEM lane = row)
//   warp 8           TMA producer (one thread)
//   warp 9           tcgen05.mma issuer (one thread); owns TMEM alloc/dealloc
//   warps 10-11      idle (they keep warpgroup 2 whole for setmaxnreg)
// TMEM, 512 columns: S0 | S1 | O0 | O1 (128 f32 columns each); the bf16
// probabilities P_i overwrite columns 0-63 of S_i and feed the P.V MMA from
// TMEM.  MMA issue order per visited key tile j: PV0(j-1) QK0(j) PV1(j-1)
// QK1(j), so one tile's softmax runs under the other tile's MMAs.
//
// Softmax: base-2 domain, running reference max m advanced LAZILY (only when
// the tile max exceeds m by more than 8, i.e. a factor 256 of headroom in P),
// so O in TMEM is rescaled a handful of times per row instead of every tile;
// the result is mathematically identical because O and l share the reference.
#pragma once
#include <cuda.h>
#include "fv_ptx.cuh"

namespace fvsdpa {

constexpr int kD = 128;
constexpr int kBN = 128;              // keys per tile
constexpr int kRowsPerCta = 256;
constexpr uint32_t kPanelB = 16384;   // 128 rows x 64 bf16, one swizzled TMA box
constexpr uint32_t kTileB = 32768;    // 128 x 128 bf16 = two panels
constexpr int kMaxSeg = 8;
constexpr int kThreads = 384;
constexpr float kLazyLog2 = 8.0f;

template <int NS>
constexpr uint32_t smem_bytes() {
    return 1024u + 2u * kTileB + (uint32_t)NS * kTileB + 256u;
}

struct Params {
    void* out;              // [bh, sq, 128] bf16 or f32
    float* lse_out;         // optional [bh, sq]: m + log2(l) in the base-2 domain, -inf for an empty row
    const float* prev_o;    // optional f32 [bh, sq, 128]: normalised result of an earlier pass over other keys
    const float* prev_lse;  // its lse (same convention); both or neither
    int* status;            // device status word (0 = fine)
    int out_is_bf16;
    int out_heads;           // 0: out is [bh, sq, 128]; h > 0: merged heads, out is [bh / h, sq, h * 128]
    int bh, sq, nqb;
    float sl2;
    int nseg;
    int seg_len[kMaxSeg];    // keys in each K/V segment
    int seg_start[kMaxSeg];  // global key index of the segment's first key
    int mask_mode;           // 0 = none, 1 = block causal
    int block_tokens, window, sink;
    int q_row0;              // global index of query row 0 (sequence-parallel shard offset)
    int heavy_first;         // walk query blocks from the last to the first
    int q_div;               // > 1: split-KV, plane i of k/v/out reads plane i / q_div of q
};

#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL) || !defined(__CUDA_ARCH__)

FV_DEV int sat_mul(int a, int b) {
    long long v = (long long)a * (long long)b;
    return v > 0x7fffffffll ? 0x7fffffff : (int)v;
}

// The key tiles a CTA visits, identical in every role.  f(seg, t, k0, lim):
// segment, tile index inside it, global index of column 0, valid columns.
template <bool MASKED, class F>
FV_DEV void walk_tiles(const Params& p, int vis_lo, int vis_hi, int vis_sink, F&& f) {
    for (int seg = 0; seg < p.nseg; seg++) {
        const int len = p.seg_len[seg], start = p.seg_start[seg];
        const int nt = (len + kBN - 1) / kBN;
        for (int t = 0; t < nt; t++) {
            const int k0 = start + t * kBN;
            const int lim = min(kBN, len - t * kBN);
            if constexpr (MASKED) {
                const int k1 = k0 + lim;
                if (!((k0 < vis_hi && k1 > vis_lo) || k0 < vis_sink)) continue;
            }
            if (!f(seg, t, k0, lim)) return;
        }
    }
}

// S (TMEM 128 x 128 f32) = Q (128 x 128, K-major SW128) . K^T (128 keys, K-major SW128): eight K=16 steps, the
// descriptors of step kk being the base ones plus a constant in the 16-byte address field (32 B per step inside a
// 64-column panel, 16 KB to the second panel).  One asm block: the issuing thread spends two adds per MMA.
FV_DEV void issue_qk(uint32_t tS, uint32_t sQ, uint32_t sK) {
    constexpr uint32_t idesc = fvp::umma_idesc_bf16(128, 128, 0);
    const uint64_t a0 = fvp::umma_desc_sw128(sQ, 16, 1024), b0 = fvp::umma_desc_sw128(sK, 16, 1024);
    asm volatile(
        "{\n\t.reg .pred pt, pf;\n\t.reg .b64 a, b;\n\t"
        "setp.ne.b32 pf, %3, %3;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
        "add.s64 a, %1, 2;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 4;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 6;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1024;\n\tadd.s64 b, %2, 1024;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1026;\n\tadd.s64 b, %2, 1026;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1028;\n\tadd.s64 b, %2, 1028;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "add.s64 a, %1, 1030;\n\tadd.s64 b, %2, 1030;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
        "}"
        ::"r"(tS), "l"(a0), "l"(b0), "r"(idesc)
        : "memory");
}
// O (TMEM 128 x 128 f32) (+)= P (TMEM bf16, 128 rows x 128 keys) . V (128 keys x 128, MN-major:
// 64-column panels kPanelB apart, 8-key groups 1024 B apart); step kk: 8 TMEM columns of P, 2 KB of V.
FV_DEV void issue_pv(uint32_t tO, uint32_t tP, uint32_t sV, bool acc) {
    constexpr uint32_t idesc = fvp::umma_idesc_bf16(128, 128, 1);
    const uint64_t b0 = fvp::umma_desc_sw128(sV, kPanelB, 1024);
    asm volatile(
        "{\n\t.reg .pred pt, p0;\n\t.reg .b64 b;\n\t.reg .b32 t;\n\t"
        "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
        "add.u32 t, %1, 8;\n\tadd.s64 b, %2, 128;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 16;\n\tadd.s64 b, %2, 256;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 24;\n\tadd.s64 b, %2, 384;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 32;\n\tadd.s64 b, %2, 512;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 40;\n\tadd.s64 b, %2, 640;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 48;\n\tadd.s64 b, %2, 768;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 56;\n\tadd.s64 b, %2, 896;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "}"
        ::"r"(tO), "r"(tP), "l"(b0), "r"(idesc), "r"((uint32_t)acc)
        : "memory");
}

// Half of issue_pv: keys 64*half .. 64*half+63 (four K=16 steps).
FV_DEV void issue_pv_part(uint32_t tO, uint32_t tP, uint32_t sV, bool acc, int half) {
    constexpr uint32_t idesc = fvp::umma_idesc_bf16(128, 128, 1);
    const uint64_t b0 = fvp::umma_desc_sw128(sV + 8192u * (uint32_t)half, kPanelB, 1024);
    const uint32_t tPh = tP + 32u * (uint32_t)half;
    asm volatile(
        "{\n\t.reg .pred pt, p0;\n\t.reg .b64 b;\n\t.reg .b32 t;\n\t"
        "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
        "add.u32 t, %1, 8;\n\tadd.s64 b, %2, 128;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 16;\n\tadd.s64 b, %2, 256;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 24;\n\tadd.s64 b, %2, 384;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "}"
        ::"r"(tO), "r"(tPh), "l"(b0), "r"(idesc), "r"((uint32_t)acc)
        : "memory");
}

FV_DEV float u2f(uint32_t u) { return __uint_as_float(u); }
FV_DEV uint32_t f2u(float f) { return __float_as_uint(f); }

// Row maximum of the 128 scores (V3: three-input max).
template <bool V3, int ABL = 0>
FV_DEV float row_max(const uint32_t (&u)[128]) {
    using namespace fvp;
    if constexpr ((ABL & 2) != 0) return u2f(u[0]);  // timing ablation only: no row maximum
    if constexpr (V3) {
        float x0 = max3(u2f(u[0]), u2f(u[1]), u2f(u[2])), x1 = max3(u2f(u[3]), u2f(u[4]), u2f(u[5]));
        float x2 = max3(u2f(u[6]), u2f(u[7]), u2f(u[8])), x3 = max3(u2f(u[9]), u2f(u[10]), u2f(u[11]));
#pragma unroll
        for (int c = 12; c < 124; c += 8) {
            x0 = max3(x0, u2f(u[c]), u2f(u[c + 1]));
            x1 = max3(x1, u2f(u[c + 2]), u2f(u[c + 3]));
            x2 = max3(x2, u2f(u[c + 4]), u2f(u[c + 5]));
            x3 = max3(x3, u2f(u[c + 6]), u2f(u[c + 7]));
        }
        x0 = max3(x0, u2f(u[124]), u2f(u[125]));
        x1 = max3(x1, u2f(u[126]), u2f(u[127]));
        return fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
    } else {
        float x0 = u2f(u[0]), x1 = u2f(u[1]), x2 = u2f(u[2]), x3 = u2f(u[3]);
#pragma unroll
        for (int c = 4; c < 128; c += 4) {
            x0 = fmaxf(x0, u2f(u[c]));
            x1 = fmaxf(x1, u2f(u[c + 1]));
            x2 = fmaxf(x2, u2f(u[c + 2]));
            x3 = fmaxf(x3, u2f(u[c + 3]));
        }
        return fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
    }
}

// P = 2^(s*sl2 + noff) for the 128 scores of one row: bf16 pairs stored to TMEM at tP, returns the f32 row sum.
// PACK: two-wide FMA / ADD.  PMASK >= 0: the pairs w of each half with (w & PMASK) == PMASK go through the
// FMA-pipe exponential (1 -> every second pair, 3 -> every fourth), the others through MUFU ex2.
template <bool PACK, int PMASK, int ABL = 0>
FV_DEV float exp_and_store(const uint32_t (&u)[128], float sl2, float noff, uint32_t tP, uint32_t bar_half = 0u) {
    using namespace fvp;
    float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
    uint64_t ya = pack_f32x2(0.f, 0.f), yb = pack_f32x2(0.f, 0.f);
    const uint64_t sl2x = pack_f32x2(sl2, sl2), noffx = pack_f32x2(noff, noff);
#pragma unroll
    for (int h = 0; h < 2; h++) {
        uint32_t pw[32];
#pragma unroll
        for (int w = 0; w < 32; w++) {
            const int c = 64 * h + 2 * w;
            float t0, t1, p0, p1;
            if constexpr (PACK) {
                unpack_f32x2(fma_f32x2(pack_f32x2(u2f(u[c]), u2f(u[c + 1])), sl2x, noffx), t0, t1);
            } else {
                t0 = fmaf(u2f(u[c]), sl2, noff);
                t1 = fmaf(u2f(u[c + 1]), sl2, noff);
            }
            if constexpr ((ABL & 1) != 0) {  // timing ablation only: no exponential
                p0 = t0;
                p1 = t1;
            } else if constexpr (PMASK >= 0) {
                if ((w & PMASK) == PMASK) {
                    ex2_poly_x2(t0, t1, p0, p1);
                } else {
                    p0 = ex2(t0);
                    p1 = ex2(t1);
                }
            } else {
                p0 = ex2(t0);
                p1 = ex2(t1);
            }
            if constexpr ((ABL & 4) != 0) {  // timing ablation only: no row sum
                if (w == 0) y0 = p0;
            } else if constexpr (PACK) {
                if (w & 1) yb = add_f32x2(yb, pack_f32x2(p0, p1));
                else ya = add_f32x2(ya, pack_f32x2(p0, p1));
            } else {
                if (w & 1) { y2 += p0; y3 += p1; }
                else { y0 += p0; y1 += p1; }
            }
            pw[w] = pack_bf16x2(p0, p1);
        }
        if constexpr ((ABL & 16) == 0) tmem_st32(tP + 32u * h, pw);  // (ABL 16: timing ablation, P is not stored)
        else if (pw[0] == 0xdeadbeefu && pw[31] == 0x12345u) tmem_st32(tP + 32u * h, pw);
        if (h == 0 && bar_half != 0u) {  // hand the first 64 keys over
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_half);
        }
    }
    if constexpr (PACK) {
        unpack_f32x2(ya, y0, y1);
        unpack_f32x2(yb, y2, y3);
    }
    return (y0 + y1) + (y2 + y3);
}

// VAR bits: 1 = packed f32x2 scale-and-subtract and row sum; 2 = half of the exponentials of an unmasked
// tile on the FMA pipe (pairs 1, 3, 5, ... of each group of four columns); 4 = a quarter of them instead;
// 8 = three-input max; 16 = exponentials against the current reference before the row maximum is known (P stored speculatively);
// 32 = the same in registers, stored only once it is known to stand, row sum after the signal.
// MASKED = false compiles the block-causal bookkeeping out (dense calls: fewer live registers in the softmax loop).
// SPLITP: P is handed to the MMA thread in two halves (keys 0-63, then 64-127), so P.V starts while the second half of
// the exponentials is still being computed.
template <int NS, int VAR, bool MASKED, bool SPLITP = false>
FV_DEV void sdpa_body(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const Params& p,
                      unsigned char* smem_raw) {
    using namespace fvp;
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t sQ = base;
    const uint32_t ring = base + 2 * kTileB;
    const uint32_t bars = ring + NS * kTileB;
    const uint32_t b_q = bars;
    const uint32_t b_full = b_q + 8;
    const uint32_t b_empty = b_full + 8 * NS;
    const uint32_t b_s = b_empty + 8 * NS;
    const uint32_t b_p = b_s + 16;
    const uint32_t b_o = b_p + 16;
    const uint32_t b_pa = b_o + 16;   // first half of P stored (SPLITP)
    const uint32_t b_drain = b_pa + 16;
    const uint32_t tslot = b_drain + 8;
    const uint32_t aflag = tslot + 4;
    volatile uint32_t* tslot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tslot - raw));
    volatile int* abort_ptr = reinterpret_cast<volatile int*>(smem_raw + (aflag - raw));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int qb = (int)(blockIdx.x % (unsigned)p.nqb);
    const int bh = (int)(blockIdx.x / (unsigned)p.nqb);
    if (p.heavy_first) qb = p.nqb - 1 - qb;
    const int q0 = qb * kRowsPerCta;
    const float NEG = __int_as_float(0xff800000);

    if (tid == 0) {
        mbar_init(b_q, 1);
        for (int i = 0; i < NS; i++) {
            mbar_init(b_full + 8 * i, 1);
            mbar_init(b_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(b_s + 8 * i, 1);
            mbar_init(b_p + 8 * i, 128);
            mbar_init(b_o + 8 * i, 1);
            mbar_init(b_pa + 8 * i, 128);
        }
        mbar_init(b_drain, 1);
        // A CTA that starts after another one gave up does nothing.
        *abort_ptr = (*(volatile int*)p.status != FV_ST_OK) ? 1 : 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (*abort_ptr) return;  // CTA-uniform
    if (warp == 9) tmem_alloc(tslot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tslot_ptr;

    // Keys any row of this CTA may see (block-causal): [vis_lo, vis_hi) U [0, vis_sink).
    int vis_lo = 0, vis_hi = 0x7fffffff, vis_sink = 0;
    const int bt = max(p.block_tokens, 1);
    if constexpr (MASKED) {
        const int qg_min = p.q_row0 + q0;
        const int qg_max = p.q_row0 + min(q0 + kRowsPerCta - 1, p.sq - 1);
        const int tq_min = qg_min / bt, tq_max = qg_max / bt;
        vis_hi = sat_mul(tq_max + 1, bt);
        vis_lo = p.window > 0 ? sat_mul(max(0, tq_min - p.window + 1), bt) : 0;
        vis_sink = sat_mul(p.sink, bt);
    }

    if (warp < 8) {
        // Register budget: the CTA's pool is what the launch allocated, 384 x 168 = 64512.
        // 256 x 224 + 128 x 56 = 64512 exactly; asking for more blocks the warpgroup forever.
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;" ::: "memory");
        // ------------------------------------------------------------ softmax
        WaitCtl ctl{abort_ptr, p.status, 3};
        const int tile = warp >> 2, sub = warp & 3;
        const int row = sub * 32 + lane;
        const uint32_t tl = tbase + ((uint32_t)(sub * 32) << 16);
        const uint32_t tS = tl + 128u * tile, tP = tS, tO = tl + 256u + 128u * tile;
        const int qr = q0 + 128 * tile + row;
        // Keys this row may see: [r_lo, r_hi) U [0, r_sink).
        int r_lo = 0, r_hi = 0x7fffffff, r_sink = 0;
        if constexpr (MASKED) {
            const int tqr = (p.q_row0 + qr) / bt;
            r_hi = sat_mul(tqr + 1, bt);
            r_lo = p.window > 0 ? sat_mul(max(0, tqr - p.window + 1), bt) : 0;
            r_sink = vis_sink;
        }
        const float sl2 = p.sl2;
        float m = NEG, l = 0.f;
        int it = 0;
        bool ok = true;
        walk_tiles<MASKED>(p, vis_lo, vis_hi, vis_sink, [&](int, int, int k0, int lim) -> bool {
            // Warp-uniform outcome: the TMEM instructions below are warp-collective.
            if (!__all_sync(0xffffffffu, mbar_wait(b_s + 8 * tile, it & 1, ctl))) { ok = false; return false; }
            tc_fence_after();
            uint32_t u[128];
            bool full_tile;
            // S of this row into registers, columns the row may not see set to -inf
            auto load_scores = [&]() {
                if constexpr (((VAR >> 6) & 8) != 0) {  // timing ablation only: S is not read
#pragma unroll
                    for (int c = 0; c < 128; c++) u[c] = 0x3f800000u + (uint32_t)c;
                    tmem_pin(u);
                } else {
                    tmem_ld32_issue<0>(tS, u);
                    tmem_ld32_issue<32>(tS + 32u, u);
                    tmem_ld32_issue<64>(tS + 64u, u);
                    tmem_ld32_issue<96>(tS + 96u, u);
                    tmem_ld_wait();
                    tmem_pin(u);
                }
                if constexpr (MASKED) {
                    // Visible columns of this row in this tile: [c_lo, c_hi) U [0, c_sink).
                    const int c_lo = min(max(r_lo - k0, 0), lim);
                    const int c_hi = min(max(r_hi - k0, 0), lim);
                    const int c_sink = min(max(r_sink - k0, 0), lim);
                    full_tile = (c_lo == 0 && c_hi == kBN) || c_sink == kBN;
                    if (!full_tile) {
#pragma unroll
                        for (int c = 0; c < 128; c++) {
                            const bool vis = (c >= c_lo && c < c_hi) || c < c_sink;
                            u[c] = vis ? u[c] : f2u(NEG);
                        }
                    }
                } else {
                    (void)k0;
                    full_tile = lim == kBN;  // only a segment's last tile can be short
                    if (!full_tile) {
#pragma unroll
                        for (int c = 0; c < 128; c++) u[c] = c < lim ? u[c] : f2u(NEG);
                    }
                }
            };
            load_scores();
            if constexpr ((VAR & 32) != 0) {
                // Fast path, taken for almost every tile after the first ones: every row of the warp has a finite
                // reference m, so P = 2^(s*sl2 - m) is computed in place in registers before anything is known about
                // this tile's maximum.  If no P exceeds 2^8 the reference stays: pack, store, signal, and only then
                // add up the row sum (nothing downstream waits for it).  Otherwise S is still intact in TMEM: read
                // it again and take the exact path below.
                if (__all_sync(0xffffffffu, m != NEG)) {
                    const float nm = -m;
                    float g0 = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f;
#pragma unroll
                    for (int c = 0; c < 128; c += 4) {
                        const float p0 = ex2(fmaf(u2f(u[c]), sl2, nm)), p1 = ex2(fmaf(u2f(u[c + 1]), sl2, nm));
                        const float p2 = ex2(fmaf(u2f(u[c + 2]), sl2, nm)), p3 = ex2(fmaf(u2f(u[c + 3]), sl2, nm));
                        g0 = fmaxf(g0, p0);
                        g1 = fmaxf(g1, p1);
                        g2 = fmaxf(g2, p2);
                        g3 = fmaxf(g3, p3);
                        u[c] = f2u(p0);
                        u[c + 1] = f2u(p1);
                        u[c + 2] = f2u(p2);
                        u[c + 3] = f2u(p3);
                    }
                    const float pmax = fmaxf(fmaxf(g0, g1), fmaxf(g2, g3));
                    if (!__any_sync(0xffffffffu, !(pmax <= 256.f))) {
#pragma unroll
                        for (int h = 0; h < 2; h++) {
                            uint32_t pw[32];
#pragma unroll
                            for (int w = 0; w < 32; w++) pw[w] = pack_bf16x2(u2f(u[64 * h + 2 * w]), u2f(u[64 * h + 2 * w + 1]));
                            tmem_st32(tP + 32u * h, pw);
                        }
                        tmem_st_wait();
                        tc_fence_before();
                        mbar_arrive(b_p + 8 * tile);
                        float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
                        for (int c = 0; c < 128; c += 4) {
                            y0 += u2f(u[c]);
                            y1 += u2f(u[c + 1]);
                            y2 += u2f(u[c + 2]);
                            y3 += u2f(u[c + 3]);
                        }
                        l += (y0 + y1) + (y2 + y3);
                        it++;
                        return true;
                    }
                    load_scores();
                }
            }
            bool settled = false;  // warp-uniform: the speculative pass below already produced this tile's P
            if constexpr ((VAR & 16) != 0) {
                // Every row of the warp already has a finite reference: exponentiate against it right away and
                // compute the row maximum beside it (independent instruction streams; the maximum only decides
                // whether the reference has to move, which is rare after the first tiles).
                if (__all_sync(0xffffffffu, m != NEG)) {
                    const float rs = exp_and_store<(VAR & 1) != 0, -1>(u, sl2, -m, tP);
                    const float t2 = row_max<(VAR & 8) != 0>(u) * sl2;
                    if (!__any_sync(0xffffffffu, t2 > m + kLazyLog2)) {
                        l += rs;
                        settled = true;
                    }
                }
            }
            if (!settled) {
            const float tmax = row_max<(VAR & 8) != 0, (VAR >> 6)>(u);
            const float tm2 = tmax * sl2;
            const bool grow = tm2 > m + kLazyLog2;
            float a = 1.f;
            if (grow) {
                a = ex2(m - tm2);
                m = tm2;
            }
            const float off = (m == NEG) ? 0.f : m;
            // O holds P.V of the tiles before this one (its MMA finished before
            // this S did): rescale it when a row of the warp moved its reference.
            if (it > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                for (int q = 0; q < 4; q++) {
                    uint32_t o[32];
                    tmem_ld32_issue(tO + 32u * q, o);
                    tmem_ld_wait();
                    tmem_pin(o);
#pragma unroll
                    for (int c = 0; c < 32; c++) o[c] = f2u(u2f(o[c]) * a);
                    tmem_st32(tO + 32u * q, o);
                }
            }
            const float noff = -off;
            constexpr int kPolyMask = (VAR & 2) ? 1 : ((VAR & 4) ? 3 : -1);
            // the FMA-pipe exponential never returns an exact zero: masked tiles keep the MUFU path
            float rowsum;
            // (warp-uniform choice: the TMEM store inside is warp-collective and must not sit in divergent code)
            if (kPolyMask >= 0 && __all_sync(0xffffffffu, full_tile))
                rowsum = exp_and_store<(VAR & 1) != 0, kPolyMask, (VAR >> 6)>(u, sl2, noff, tP, SPLITP ? b_pa + 8 * tile : 0u);
            else rowsum = exp_and_store<(VAR & 1) != 0, -1, (VAR >> 6)>(u, sl2, noff, tP, SPLITP ? b_pa + 8 * tile : 0u);
            l = fmaf(l, a, rowsum);
            }
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(b_p + 8 * tile);
            it++;
            return true;
        });

        // ----------------------------------------------------------- epilogue
        if (ok && it > 0) ok = __all_sync(0xffffffffu, mbar_wait(b_o + 8 * tile, 0, ctl));
        tc_fence_after();
        if (ok) {
            const bool live = qr < p.sq;  // rows past sq take part in the warp-collective TMEM loads only
            float inv = l > 0.f ? 1.f / l : 0.f;
            const float lse = l > 0.f ? m + log2f(l) : NEG;
            const size_t rowi = (size_t)bh * p.sq + (live ? qr : 0);
            float cp = 0.f;  // weight of the earlier pass
            if (live) {
                if (p.prev_o) {
                    const float pl = p.prev_lse[rowi];
                    const float M = fmaxf(lse, pl);
                    float lse_all = NEG;
                    if (M != NEG) {
                        const float wn = exp2f(lse - M), wp = exp2f(pl - M);
                        const float den = 1.f / (wn + wp);
                        inv *= wn * den;
                        cp = wp * den;
                        lse_all = M + log2f(wn + wp);
                    }
                    if (p.lse_out) p.lse_out[rowi] = lse_all;
                } else if (p.lse_out) {
                    p.lse_out[rowi] = lse;
                }
            }
            const size_t off = rowi * kD;  // BHSD offset (earlier pass, lse)
            size_t ooff = off;             // where this row's output goes
            if (p.out_heads > 0) {
                const int bb = bh / p.out_heads, hh = bh % p.out_heads;
                ooff = (((size_t)bb * p.sq + (live ? qr : 0)) * p.out_heads + hh) * kD;
            }
#pragma unroll 1
            for (int q = 0; q < 4; q++) {
                uint32_t o[32];
                if (it > 0) {  // CTA-uniform
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
                for (int c = 0; c < 32; c++) f[c] = u2f(o[c]) * inv;
                if (p.prev_o) {
                    const float4* po = reinterpret_cast<const float4*>(p.prev_o + off + 32 * q);
#pragma unroll
                    for (int c = 0; c < 8; c++) {
                        const float4 t = po[c];
                        f[4 * c] = fmaf(t.x, cp, f[4 * c]);
                        f[4 * c + 1] = fmaf(t.y, cp, f[4 * c + 1]);
                        f[4 * c + 2] = fmaf(t.z, cp, f[4 * c + 2]);
                        f[4 * c + 3] = fmaf(t.w, cp, f[4 * c + 3]);
                    }
                }
                if (p.out_is_bf16) {
                    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(p.out) + ooff + 32 * q);
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        dst[c] = make_uint4(pack_bf16x2(f[8 * c], f[8 * c + 1]), pack_bf16x2(f[8 * c + 2], f[8 * c + 3]),
                                            pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), pack_bf16x2(f[8 * c + 6], f[8 * c + 7]));
                } else {
                    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + ooff + 32 * q);
#pragma unroll
                    for (int c = 0; c < 8; c++) dst[c] = make_float4(f[4 * c], f[4 * c + 1], f[4 * c + 2], f[4 * c + 3]);
                }
            }
        }
        // Every TMEM access of this thread is complete: warp 9 may free the columns.
        tc_fence_before();
        asm volatile("bar.arrive 1, 288;" ::: "memory");
        return;
    }

    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == 8) {
        // ------------------------------------------------------- TMA producer
        if (lane == 0) {
            WaitCtl ctl{abort_ptr, p.status, 1};
            tma_prefetch_desc(tq);
            tma_prefetch_desc(tk);
            tma_prefetch_desc(tv);
            mbar_expect_tx(b_q, 2 * kTileB);
            const int bhq = p.q_div > 1 ? bh / p.q_div : bh;
            tma_load4(sQ, tq, b_q, 0, q0, bhq, 0);
            tma_load4(sQ + kPanelB, tq, b_q, 64, q0, bhq, 0);
            tma_load4(sQ + kTileB, tq, b_q, 0, q0 + 128, bhq, 0);
            tma_load4(sQ + kTileB + kPanelB, tq, b_q, 64, q0 + 128, bhq, 0);
            int idx = 0;
            bool ok = true;
            walk_tiles<MASKED>(p, vis_lo, vis_hi, vis_sink, [&](int seg, int t, int, int) -> bool {
#pragma unroll 1
                for (int half = 0; half < 2; half++) {
                    const int slot = idx % NS, use = idx / NS;
                    if (use > 0 && !mbar_wait(b_empty + 8 * slot, (use - 1) & 1, ctl)) { ok = false; return false; }
                    const uint32_t dst = ring + slot * kTileB, bar = b_full + 8 * slot;
                    const CUtensorMap* map = half ? tv : tk;
                    if (((VAR >> 6) & 128) != 0 && idx >= NS) {  // timing ablation only: the ring is not refilled
                        mbar_arrive(bar);
                    } else {
                        mbar_expect_tx(bar, kTileB);
                        tma_load4(dst, map, bar, 0, t * kBN, bh, seg);
                        tma_load4(dst + kPanelB, map, bar, 64, t * kBN, bh, seg);
                    }
                    idx++;
                }
                return true;
            });
            // Copies in flight must land before the CTA's shared memory goes away.  On the
            // normal path the MMA thread has already waited on each of these phases.
            mbar_wait(b_q, 0, ctl);
            for (int s = 0; s < NS && s < idx; s++) {
                const int last = ((idx - 1 - s) / NS) * NS + s;  // last load index that used slot s
                mbar_wait(b_full + 8 * s, (last / NS) & 1, ctl);
            }
            (void)ok;
        }
        return;
    }
    if (warp == 9) {
        // --------------------------------------------------------- MMA issuer
        if (lane == 0) {
            WaitCtl ctl{abort_ptr, p.status, 2};
            // This role needs only the number of visited tiles, not which ones.
            int nvis = 0;
            walk_tiles<MASKED>(p, vis_lo, vis_hi, vis_sink, [&](int, int, int, int) -> bool { nvis++; return true; });
            bool ok = mbar_wait(b_q, 0, ctl);
            tc_fence_after();
            int it = 0;
#pragma unroll 1
            for (; ok && it < nvis; it++) {
                const int ik = 2 * it, slotK = ik % NS;
                if (!mbar_wait(b_full + 8 * slotK, (ik / NS) & 1, ctl)) { ok = false; break; }
                tc_fence_after();
                const uint32_t sK = ring + slotK * kTileB;
                if (it == 0) {
                    issue_qk(tbase, sQ, sK);
                    umma_commit(b_s);
                    issue_qk(tbase + 128u, sQ + kTileB, sK);
                    umma_commit(b_s + 8);
                    umma_commit(b_empty + 8 * slotK);
                } else {
                    const int iv = ik - 1, slotV = iv % NS;
                    if (!mbar_wait(b_full + 8 * slotV, (iv / NS) & 1, ctl)) { ok = false; break; }
                    const uint32_t sV = ring + slotV * kTileB;
#pragma unroll
                    for (int i = 0; i < 2; i++) {
                        if constexpr (SPLITP) {
                            if (ok && !mbar_wait(b_pa + 8 * i, (it - 1) & 1, ctl)) ok = false;
                            if (ok) {
                                tc_fence_after();
                                issue_pv_part(tbase + 256u + 128u * i, tbase + 128u * i, sV, it > 1, 0);
                            }
                        }
                        if (ok && !mbar_wait(b_p + 8 * i, (it - 1) & 1, ctl)) ok = false;
                        if (ok) {
                            tc_fence_after();
                            if constexpr (SPLITP) issue_pv_part(tbase + 256u + 128u * i, tbase + 128u * i, sV, true, 1);
                            else if constexpr (((VAR >> 6) & 64) == 0) issue_pv(tbase + 256u + 128u * i, tbase + 128u * i, sV, it > 1);
                            if constexpr (((VAR >> 6) & 32) == 0) issue_qk(tbase + 128u * i, sQ + i * kTileB, sK);
                            umma_commit(b_s + 8 * i);
                        }
                    }
                    if (!ok) break;
                    umma_commit(b_empty + 8 * slotV);
                    umma_commit(b_empty + 8 * slotK);
                }
            }
            if (ok && it > 0) {
                const int iv = 2 * it - 1, slotV = iv % NS;
                ok = mbar_wait(b_full + 8 * slotV, (iv / NS) & 1, ctl);
                const uint32_t sV = ring + slotV * kTileB;
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    if constexpr (SPLITP) {
                        if (ok) ok = mbar_wait(b_pa + 8 * i, (it - 1) & 1, ctl);
                        if (ok) {
                            tc_fence_after();
                            issue_pv_part(tbase + 256u + 128u * i, tbase + 128u * i, sV, it > 1, 0);
                        }
                    }
                    if (ok) ok = mbar_wait(b_p + 8 * i, (it - 1) & 1, ctl);
                    if (ok) {
                        tc_fence_after();
                        if constexpr (SPLITP) issue_pv_part(tbase + 256u + 128u * i, tbase + 128u * i, sV, true, 1);
                        else issue_pv(tbase + 256u + 128u * i, tbase + 128u * i, sV, it > 1);
                        umma_commit(b_o + 8 * i);
                    }
                }
            }
            // Nothing this thread issued may still be running when TMEM is freed.
            umma_commit(b_drain);
            mbar_wait(b_drain, 0, ctl);
        }
        __syncwarp();
        asm volatile("bar.sync 1, 288;" ::: "memory");
        tc_fence_after();
        tmem_dealloc(tbase, 512);
    }
}

#endif  // sm_100a / host pass

}  // namespace fvsdpa

// Second schedule of the head-dim-128 SDPA forward: the same CTA (256 query rows, two M=128 tiles, 12 warps,
// K/V ring of 128-key tiles) with the score accumulator of each query tile DOUBLE-BUFFERED over 64-key half
// steps, so that a tile's softmax never waits for its own MMAs.
//
// TMEM, 512 columns: S0a | S0b | S1a | S1b (64 f32 columns each) | O0 | O1 (128 each).  For query tile i the MMA
// thread keeps S_i two half steps ahead: while the softmax warps work on S_i(h) in buffer h&1, S_i(h+1) is
// already computed in the other buffer, and Q.K^T of half h+2 is issued into buffer h&1 right behind P_i(h).V
// (which reads the bf16 P_i(h) stored over the first 32 columns of that buffer; same issuing thread, so in order).
// With one S buffer per tile (sdpa_fwd.cuh) every step of a tile is softmax -> own P.V -> own Q.K^T -> softmax,
// and the tensor pipe idles while a tile's softmax runs unless the other tile happens to have work queued;
// measured there: tensor pipe 52 % busy.  Here the per-tile chain is softmax -> softmax -> ...
//
// Everything else is shared with sdpa_fwd.cuh: Params, the tile walk (as a cursor), lazy rescale, block-causal
// masks, K/V segments, two-pass merge, bounded waits with a status word.
#pragma once
#include "sdpa_fwd.cuh"

namespace fvsdpa {

#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL) || !defined(__CUDA_ARCH__)

// The visited key tiles as an explicit cursor (several can be live at once), then cut into 64-key halves:
// half 1 of a tile exists when the tile holds more than 64 keys.
template <bool MASKED>
struct HalfCursor {
    int seg, t, it;   // segment, tile inside it, ordinal of the visited tile (ring slots follow it)
    int k0, lim;      // global index of the tile's first key, keys in the tile
    int hh, h;        // half inside the tile, ordinal of the half
    bool valid;
    int vis_lo, vis_hi, vis_sink;

    FV_DEV void init(const Params& p, int lo, int hi, int sink) {
        seg = 0; t = -1; it = -1; hh = 0; h = -1; k0 = 0; lim = 0;
        vis_lo = lo; vis_hi = hi; vis_sink = sink;
        valid = next_tile(p);
        if (valid) h = 0;
    }
    FV_DEV bool next_tile(const Params& p) {
        for (;;) {
            if (seg >= p.nseg) return false;
            const int len = p.seg_len[seg];
            t++;
            if (t * kBN >= len) { seg++; t = -1; continue; }
            k0 = p.seg_start[seg] + t * kBN;
            lim = min(kBN, len - t * kBN);
            if constexpr (MASKED) {
                const int k1 = k0 + lim;
                if (!((k0 < vis_hi && k1 > vis_lo) || k0 < vis_sink)) continue;
            }
            it++;
            hh = 0;
            return true;
        }
    }
    FV_DEV bool last_half_of_tile() const { return hh == 1 || lim <= 64; }
    FV_DEV void next(const Params& p) {
        if (!valid) return;
        if (hh == 0 && lim > 64) { hh = 1; h++; return; }
        valid = next_tile(p);
        if (valid) h++;
    }
};

// S half (TMEM 128 x 64 f32) = Q (128 x 128) . K^T (64 keys: rows 64*hh.. of the K tile)
FV_DEV void issue_qk_half(uint32_t tS, uint32_t sQ, uint32_t sK, int hh) {
    constexpr uint32_t idesc = fvp::umma_idesc_bf16(128, 64, 0);
    const uint64_t a0 = fvp::umma_desc_sw128(sQ, 16, 1024), b0 = fvp::umma_desc_sw128(sK + (uint32_t)hh * 8192u, 16, 1024);
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
// O (TMEM 128 x 128 f32) (+)= P (TMEM bf16 128 x 64 keys) . V (keys 64*hh.. of the V tile, 64 x 128, MN-major)
FV_DEV void issue_pv_half(uint32_t tO, uint32_t tP, uint32_t sV, int hh, bool acc) {
    constexpr uint32_t idesc = fvp::umma_idesc_bf16(128, 128, 1);
    const uint64_t b0 = fvp::umma_desc_sw128(sV + 8192u * (uint32_t)hh, kPanelB, 1024);
    asm volatile(
        "{\n\t.reg .pred pt, p0;\n\t.reg .b64 b;\n\t.reg .b32 t;\n\t"
        "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
        "add.u32 t, %1, 8;\n\tadd.s64 b, %2, 128;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 16;\n\tadd.s64 b, %2, 256;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "add.u32 t, %1, 24;\n\tadd.s64 b, %2, 384;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
        "}"
        ::"r"(tO), "r"(tP), "l"(b0), "r"(idesc), "r"((uint32_t)acc)
        : "memory");
}

// VAR bits: 1 = P against the current reference before the half's maximum is known (in registers; stored only if
// it stands), row sum after the signal.
template <int NS, int VAR, bool MASKED>
FV_DEV void sdpa_body64(const CUtensorMap* tq, const CUtensorMap* tk, const CUtensorMap* tv, const Params& p,
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
    const uint32_t b_s = b_empty + 8 * NS;   // [tile][buf]
    const uint32_t b_p = b_s + 32;           // [tile][buf]
    const uint32_t b_od = b_p + 32;          // [tile]: one phase per P.V
    const uint32_t b_o = b_od + 16;          // [tile]: the last P.V
    const uint32_t b_drain = b_o + 16;
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
        for (int i = 0; i < 4; i++) {
            mbar_init(b_s + 8 * i, 1);
            mbar_init(b_p + 8 * i, 128);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(b_od + 8 * i, 1);
            mbar_init(b_o + 8 * i, 1);
        }
        mbar_init(b_drain, 1);
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
        asm volatile("setmaxnreg.inc.sync.aligned.u32 224;" ::: "memory");  // 256*224 + 128*56 = 384*168
        // ------------------------------------------------------------ softmax
        WaitCtl ctl{abort_ptr, p.status, 3};
        const int tile = warp >> 2, sub = warp & 3;
        const int row = sub * 32 + lane;
        const uint32_t tl = tbase + ((uint32_t)(sub * 32) << 16);
        const uint32_t tS = tl + 128u * tile, tO = tl + 256u + 128u * tile;
        const int qr = q0 + 128 * tile + row;
        int r_lo = 0, r_hi = 0x7fffffff, r_sink = 0;
        if constexpr (MASKED) {
            const int tqr = (p.q_row0 + qr) / bt;
            r_hi = sat_mul(tqr + 1, bt);
            r_lo = p.window > 0 ? sat_mul(max(0, tqr - p.window + 1), bt) : 0;
            r_sink = vis_sink;
        }
        const float sl2 = p.sl2;
        float m = NEG, l = 0.f;
        bool ok = true;
        HalfCursor<MASKED> cur;
        cur.init(p, vis_lo, vis_hi, vis_sink);
        int nhalf = 0;
#pragma unroll 1
        for (; cur.valid; cur.next(p)) {
            const int h = cur.h, b = h & 1;
            nhalf = h + 1;
            const uint32_t tSb = tS + 64u * b;
            const uint32_t bar_s = b_s + 8 * (2 * tile + b), bar_p = b_p + 8 * (2 * tile + b);
            if (!__all_sync(0xffffffffu, mbar_wait(bar_s, (h >> 1) & 1, ctl))) { ok = false; break; }
            tc_fence_after();
            const int kh = cur.k0 + 64 * cur.hh;            // global index of column 0 of this half
            const int limh = min(64, cur.lim - 64 * cur.hh);  // keys in this half
            uint32_t u[64];
            auto load_scores = [&]() {
                {
                    uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&u[0]);
                    uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&u[32]);
                    tmem_ld32_issue(tSb, lo);
                    tmem_ld32_issue(tSb + 32u, hi);
                }
                tmem_ld_wait();
                tmem_pin(u);
                if constexpr (MASKED) {
                    const int c_lo = min(max(r_lo - kh, 0), limh);
                    const int c_hi = min(max(r_hi - kh, 0), limh);
                    const int c_sink = min(max(r_sink - kh, 0), limh);
                    if (!((c_lo == 0 && c_hi == 64) || c_sink == 64)) {
#pragma unroll
                        for (int c = 0; c < 64; c++) {
                            const bool vis = (c >= c_lo && c < c_hi) || c < c_sink;
                            u[c] = vis ? u[c] : f2u(NEG);
                        }
                    }
                } else {
                    if (limh < 64) {
#pragma unroll
                        for (int c = 0; c < 64; c++) u[c] = c < limh ? u[c] : f2u(NEG);
                    }
                }
            };
            load_scores();
            bool settled = false;
            if constexpr ((VAR & 1) != 0) {
                if (__all_sync(0xffffffffu, m != NEG)) {
                    const float nm = -m;
                    float g0 = 0.f, g1 = 0.f, g2 = 0.f, g3 = 0.f;
#pragma unroll
                    for (int c = 0; c < 64; c += 4) {
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
                        uint32_t pw[32];
#pragma unroll
                        for (int w = 0; w < 32; w++) pw[w] = pack_bf16x2(u2f(u[2 * w]), u2f(u[2 * w + 1]));
                        tmem_st32(tSb, pw);
                        tmem_st_wait();
                        tc_fence_before();
                        mbar_arrive(bar_p);
                        float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
                        for (int c = 0; c < 64; c += 4) {
                            y0 += u2f(u[c]);
                            y1 += u2f(u[c + 1]);
                            y2 += u2f(u[c + 2]);
                            y3 += u2f(u[c + 3]);
                        }
                        l += (y0 + y1) + (y2 + y3);
                        settled = true;
                    } else {
                        load_scores();  // S is still intact in TMEM
                    }
                }
            }
            if (settled) continue;
            float x0 = u2f(u[0]), x1 = u2f(u[1]), x2 = u2f(u[2]), x3 = u2f(u[3]);
#pragma unroll
            for (int c = 4; c < 64; c += 4) {
                x0 = fmaxf(x0, u2f(u[c]));
                x1 = fmaxf(x1, u2f(u[c + 1]));
                x2 = fmaxf(x2, u2f(u[c + 2]));
                x3 = fmaxf(x3, u2f(u[c + 3]));
            }
            const float tm2 = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3)) * sl2;
            const bool grow = tm2 > m + kLazyLog2;
            float a = 1.f;
            if (grow) {
                a = ex2(m - tm2);
                m = tm2;
            }
            const float off = (m == NEG) ? 0.f : m;
            if (h > 0 && __any_sync(0xffffffffu, grow)) {
                // O must be quiet: P.V of half h-1 may still be running (S of this half only implies h-2 is done).
                if (!__all_sync(0xffffffffu, mbar_wait(b_od + 8 * tile, (h - 1) & 1, ctl))) { ok = false; break; }
                tc_fence_after();
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
            float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
            {
                uint32_t pw[32];
#pragma unroll
                for (int w = 0; w < 32; w += 2) {
                    const float p0 = ex2(fmaf(u2f(u[2 * w]), sl2, -off)), p1 = ex2(fmaf(u2f(u[2 * w + 1]), sl2, -off));
                    const float p2 = ex2(fmaf(u2f(u[2 * w + 2]), sl2, -off)), p3 = ex2(fmaf(u2f(u[2 * w + 3]), sl2, -off));
                    y0 += p0;
                    y1 += p1;
                    y2 += p2;
                    y3 += p3;
                    pw[w] = pack_bf16x2(p0, p1);
                    pw[w + 1] = pack_bf16x2(p2, p3);
                }
                tmem_st32(tSb, pw);
            }
            l = fmaf(l, a, (y0 + y1) + (y2 + y3));
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bar_p);
        }

        // ----------------------------------------------------------- epilogue
        if (ok && nhalf > 0) ok = __all_sync(0xffffffffu, mbar_wait(b_o + 8 * tile, 0, ctl));
        tc_fence_after();
        if (ok) {
            const bool live = qr < p.sq;
            float inv = l > 0.f ? 1.f / l : 0.f;
            const float lse = l > 0.f ? m + log2f(l) : NEG;
            const size_t rowi = (size_t)bh * p.sq + (live ? qr : 0);
            float cp = 0.f;
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
                if (nhalf > 0) {  // CTA-uniform
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
        tc_fence_before();
        asm volatile("bar.arrive 1, 288;" ::: "memory");
        return;
    }

    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;" ::: "memory");
    if (warp == 8) {
        // ------------------------------------------------------- TMA producer (whole 128-key tiles, K0 V0 K1 V1 ...)
        if (lane == 0) {
            WaitCtl ctl{abort_ptr, p.status, 1};
            tma_prefetch_desc(tq);
            tma_prefetch_desc(tk);
            tma_prefetch_desc(tv);
            mbar_expect_tx(b_q, 2 * kTileB);
            tma_load4(sQ, tq, b_q, 0, q0, bh, 0);
            tma_load4(sQ + kPanelB, tq, b_q, 64, q0, bh, 0);
            tma_load4(sQ + kTileB, tq, b_q, 0, q0 + 128, bh, 0);
            tma_load4(sQ + kTileB + kPanelB, tq, b_q, 64, q0 + 128, bh, 0);
            int idx = 0;
            walk_tiles<MASKED>(p, vis_lo, vis_hi, vis_sink, [&](int seg, int t, int, int) -> bool {
#pragma unroll 1
                for (int half = 0; half < 2; half++) {
                    const int slot = idx % NS, use = idx / NS;
                    if (use > 0 && !mbar_wait(b_empty + 8 * slot, (use - 1) & 1, ctl)) return false;
                    const uint32_t dst = ring + slot * kTileB, bar = b_full + 8 * slot;
                    const CUtensorMap* map = half ? tv : tk;
                    mbar_expect_tx(bar, kTileB);
                    tma_load4(dst, map, bar, 0, t * kBN, bh, seg);
                    tma_load4(dst + kPanelB, map, bar, 64, t * kBN, bh, seg);
                    idx++;
                }
                return true;
            });
            mbar_wait(b_q, 0, ctl);
            for (int s = 0; s < NS && s < idx; s++) {
                const int last = ((idx - 1 - s) / NS) * NS + s;
                mbar_wait(b_full + 8 * s, (last / NS) & 1, ctl);
            }
        }
        return;
    }
    if (warp == 9) {
        // --------------------------------------------------------- MMA issuer
        if (lane == 0) {
            WaitCtl ctl{abort_ptr, p.status, 2};
            bool ok = mbar_wait(b_q, 0, ctl);
            tc_fence_after();
            HalfCursor<MASKED> hq, hp;  // the half whose Q.K^T is issued next (two ahead), the half whose P.V is next
            hq.init(p, vis_lo, vis_hi, vis_sink);
            hp.init(p, vis_lo, vis_hi, vis_sink);
            // Q.K^T of half hq for query tile i into its buffer; K tile = ring index 2*it.
            auto qk = [&](int i) -> bool {
                const int ik = 2 * hq.it, slot = ik % NS;
                if (!mbar_wait(b_full + 8 * slot, (ik / NS) & 1, ctl)) return false;
                tc_fence_after();
                const int b = hq.h & 1;
                issue_qk_half(tbase + 128u * i + 64u * b, sQ + i * kTileB, ring + slot * kTileB, hq.hh);
                umma_commit(b_s + 8 * (2 * i + b));
                return true;
            };
            auto qk_done = [&]() {  // both tiles issued half hq: release the K tile after its last half
                if (hq.last_half_of_tile()) umma_commit(b_empty + 8 * ((2 * hq.it) % NS));
                hq.next(p);
            };
            // prologue: halves 0 and 1 of both tiles
            for (int n = 0; n < 2 && ok && hq.valid; n++) {
                ok = qk(0) && qk(1);
                if (ok) qk_done();
            }
            bool any = false;
#pragma unroll 1
            for (; ok && hp.valid; hp.next(p)) {
                any = true;
                const int h = hp.h, b = h & 1;
                const int iv = 2 * hp.it + 1, slotV = iv % NS;
                if (!mbar_wait(b_full + 8 * slotV, (iv / NS) & 1, ctl)) { ok = false; break; }
                const uint32_t sV = ring + slotV * kTileB;
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    if (ok && !mbar_wait(b_p + 8 * (2 * i + b), (h >> 1) & 1, ctl)) ok = false;
                    if (!ok) break;
                    tc_fence_after();
                    issue_pv_half(tbase + 256u + 128u * i, tbase + 128u * i + 64u * b, sV, hp.hh, h > 0);
                    umma_commit(b_od + 8 * i);
                    if (hq.valid) ok = qk(i);  // half h+2 into the buffer P.V(h) just read
                }
                if (!ok) break;
                if (hp.last_half_of_tile()) umma_commit(b_empty + 8 * slotV);
                if (hq.valid) qk_done();
            }
            if (ok && any) {
                umma_commit(b_o);
                umma_commit(b_o + 8);
            }
            umma_commit(b_drain);
            mbar_wait(b_drain, 0, ctl);
        }
        __syncwarp();
        asm volatile("bar.sync 1, 288;" ::: "memory");
        tc_fence_after();
        tmem_dealloc(tbase, 512);
    }
}

#endif

}  // namespace fvsdpa

// Persistent flash-attention forward for head dim 128 on sm_100a.
//
// Operand convention of the launcher it replaces (crates/fastvideo-cudarc/src/rt/attn_dc.rs:213-273,
// dense_fwd, and the block-causal launcher crates/fastvideo-cudarc/src/rt/attn.rs:647-730): bf16
// [planes, s, 128] in, bf16 or f32 [planes, sq, 128] out, scores scaled by sl2 = scale * log2 e.
//
// Shape of the kernel
// -------------------
// * One CTA per SM for the whole launch.  Work items (256 query rows of one plane = two 128-row
//   accumulator tiles, "A" and "B") are dealt round-robin: CTA c takes items c, c + grid, ...
//   Under a causal mask the items of a plane are ordered heaviest first.
// * 20 warps.  The launch gives every thread 96 registers; the four softmax warpgroups then take 104
//   each and the fifth warpgroup (loader, issuer, two idle warps) drops to 64: 512 x 104 + 128 x 64
//   is exactly the 640 x 96 the CTA owns.
//     warps 0-15   softmax.  Warp w serves row tile w / 8, score columns 64 * ((w / 4) % 2) .. + 63,
//                  TMEM lanes 32 * (w % 4) .. + 31: TWO threads share a query row, each holding half
//                  of its 128 scores.  The two warps of a row sit on the same scheduler, so the MUFU
//                  and FMA latencies of one half hide under the other; the time from "S complete" to
//                  "P complete", which bounds the tensor pipe in a two-tile ping-pong, is about half
//                  of what one thread per row needs.
//     warp 16      loader: one thread issues every TMA copy (Q ring of 3 x 32 KB, K/V ring of
//                  4 x 32 KB) and runs one item ahead with the Q tiles.
//     warp 17      issuer: one thread issues every tcgen05.mma; the warp owns the TMEM allocation.
// * TMEM (512 columns): row tile t owns columns 256 t .. 256 t + 255: scores S at +0 (128 f32
//   columns), output accumulator O at +128.  The bf16 probabilities of half h overwrite the first
//   32 of that half's own 64 score columns (+64 h .. +64 h + 31), so neither thread of a row ever
//   touches a column the other one still has to read.
// * Per key tile j the issuer runs, for t = A then B:  O_t += P_t(j-1) . V(j-1);  S_t = Q_t . K(j)^T.
//   P is handed over in two steps (the first 32 keys of each half, then the rest), so the first four
//   K=16 slices of P.V start while the second half of the exponentials is still being evaluated.
// * Softmax in the base-2 domain with a LAZY reference: the per-row reference m only moves when a
//   tile's maximum exceeds it by more than 2^8, in which case O (TMEM) and the row sum are rescaled.
//   The two threads of a row agree on the tile maximum through 2 bytes of shared memory each (the
//   maximum rounded UP to bf16: any common reference at or above the true maximum is exact) and one
//   64-thread mbarrier phase; the row sums are added once per item.
// * Every wait is bounded (fv_ptx.cuh): a role that gives up records a code in the status word,
//   raises the CTA's abort flag, and every role falls through to the common exit, where copies in
//   flight are awaited, the issuer's last MMA is awaited and TMEM is freed.  No trap, no endless spin.
#pragma once
#include <cuda.h>
#include "fv_ptx.cuh"

#define FV_ST_BAD_SMEM 90  // dynamic shared memory is not 1024-byte aligned (the swizzled tiles need it)

namespace fvattn {

constexpr int kD = 128;
constexpr int kKeyTile = 128;   // keys per score tile: N of Q.K^T, K extent of P.V
constexpr int kRowTile = 128;   // query rows per accumulator: M of both products
constexpr int kItemRows = 256;  // one work item = row tiles A and B
constexpr int kWarps = 20;          // registers are allotted per four warps: 18 would be charged as 20
constexpr int kThreads = kWarps * 32;
constexpr int kSoftmaxWarps = 16;
constexpr int kLoaderWarp = 16;
constexpr int kIssuerWarp = 17;
constexpr int kQSlots = 3;
constexpr int kKvSlots = 4;
constexpr uint32_t kSlotBytes = 32768;   // 128 rows x 128 bf16: two 64-column swizzled panels
constexpr uint32_t kPanelBytes = 16384;
constexpr int kMaxSeg = 16;
constexpr float kSlackLog2 = 8.0f;
constexpr uint32_t kFullWarp = 0xffffffffu;

// Shared-memory map, offsets from the (1024-byte aligned) start of dynamic shared memory.
struct Smem {
    static constexpr uint32_t q = 0;
    static constexpr uint32_t kv = q + kQSlots * kSlotBytes;
    static constexpr uint32_t xch = kv + kKvSlots * kSlotBytes;  // u16 [row tile 2][parity 2][half 2][row 128]
    static constexpr uint32_t q_full = xch + 2048;               // mbarriers, 8 bytes each
    static constexpr uint32_t q_free = q_full + 8 * kQSlots;
    static constexpr uint32_t kv_full = q_free + 8 * kQSlots;
    static constexpr uint32_t kv_free = kv_full + 8 * kKvSlots;
    static constexpr uint32_t s_ready = kv_free + 8 * kKvSlots;  // [2] S_t complete (issuer -> softmax)
    static constexpr uint32_t p_early = s_ready + 16;            // [2] first 32 keys of each half of P_t stored
    static constexpr uint32_t p_ready = p_early + 16;            // [2] all of P_t stored
    static constexpr uint32_t o_ready = p_ready + 16;            // [2] O_t of the item complete
    static constexpr uint32_t pair = o_ready + 16;               // [8] the two warps of a (row tile, lane quarter)
    static constexpr uint32_t drain = pair + 64;
    static constexpr uint32_t tmem_slot = drain + 8;
    static constexpr uint32_t abort_flag = tmem_slot + 4;
    static constexpr uint32_t total = abort_flag + 4;
};
static_assert(Smem::total <= 232448, "more shared memory than one CTA may have");

struct Job {
    void* out;              // [planes, sq, 128] bf16 or f32 (or merged heads, see out_heads)
    float* lse_out;         // optional [planes, sq]: reference + log2(row sum), base-2 domain; -inf for an empty row
    const float* prev_o;    // optional f32 [planes, sq, 128]: normalised result of an earlier pass over other keys
    const float* prev_lse;  // its lse (same convention); both or neither
    int* status;            // device status word (0 = fine)
    int out_is_bf16;
    int out_heads;          // 0: out is [planes, sq, 128]; h > 0: out is [planes / h, sq, h * 128]
    int planes, sq, q_blocks, items;
    float sl2;
    int nseg;
    int seg_len[kMaxSeg];    // keys in each K/V segment
    int seg_start[kMaxSeg];  // global key index of the segment's first key
    int block_tokens, window, sink;  // block-causal mask parameters (MASKED kernels only)
    int q_row0;              // global index of query row 0 (sequence-parallel shard offset)
    int q_split, q_row1;     // q_split > 0: rows from q_split on are a second run whose first row has global index q_row1
                             // (a rank of a zig-zag sequence split holds an early and a late run of the sequence)
    int heavy_first;         // items of a plane from the last query block to the first
    int q_div;               // > 1: split-KV, plane i of k / v / out reads plane i / q_div of q
    long long wait_cycles;   // budget of every bounded wait
};

#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL) || !defined(__CUDA_ARCH__)

using namespace fvp;

FV_DEV float neg_inf() { return __int_as_float(0xff800000); }
FV_DEV float as_f(uint32_t u) { return __uint_as_float(u); }
FV_DEV uint32_t as_u(float f) { return __float_as_uint(f); }

FV_DEV int mul_sat(int a, int b) {
    const long long v = (long long)a * (long long)b;
    return v > 0x7fffffffll ? 0x7fffffff : (int)v;
}

// Keys a run of query rows may see under the block-causal mask (rt/attn.rs:448-453):
// [lo, hi) U [0, sink), in global key indices.
struct Span {
    int lo, hi, sink;
    FV_DEV bool touches(int k0, int k1) const { return (k0 < hi && k1 > lo) || k0 < sink; }
};
template <bool MASKED>
FV_DEV Span span_of(const Job& jb, int first_row, int last_row) {
    if constexpr (!MASKED) return Span{0, 0x7fffffff, 0};
    // (an item that straddles the two runs of a zig-zag shard has its first row in the early run and its last
    // row in the late one, so [lo of the first, hi of the last) still covers every row of it)
    const int bt = max(jb.block_tokens, 1);
    const int b0 = min(first_row, last_row) / bt, b1 = max(first_row, last_row) / bt;
    Span s;
    s.hi = mul_sat(b1 + 1, bt);
    s.lo = jb.window > 0 ? mul_sat(max(0, b0 - jb.window + 1), bt) : 0;
    s.sink = mul_sat(jb.sink, bt);
    return s;
}

// Global index (the one the mask sees) of row r of the plane.
FV_DEV int global_row(const Job& jb, int r) {
    return (jb.q_split > 0 && r >= jb.q_split) ? jb.q_row1 + (r - jb.q_split) : jb.q_row0 + r;
}

struct Item {
    int plane, q0;
};
FV_DEV Item item_at(const Job& jb, int i) {
    Item it;
    it.plane = i / jb.q_blocks;
    int qb = i - it.plane * jb.q_blocks;
    if (jb.heavy_first) qb = jb.q_blocks - 1 - qb;
    it.q0 = qb * kItemRows;
    return it;
}

// The key tiles an item visits, in the order every role walks them.
struct KeyTile {
    int seg, t, k0, valid;  // segment, tile inside it, global index of column 0, real columns
};
template <bool MASKED>
struct KeyWalk {
    int seg = 0, t = -1;
    FV_DEV bool next(const Job& jb, const Span& sp, KeyTile& out) {
        while (seg < jb.nseg) {
            ++t;
            const int len = jb.seg_len[seg];
            const int off = t * kKeyTile;
            if (off >= len) {
                ++seg;
                t = -1;
                continue;
            }
            const int k0 = jb.seg_start[seg] + off;
            const int valid = min(kKeyTile, len - off);
            if constexpr (MASKED) {
                if (!sp.touches(k0, k0 + valid)) continue;
            }
            out = KeyTile{seg, t, k0, valid};
            return true;
        }
        return false;
    }
};
template <bool MASKED>
FV_DEV int count_tiles(const Job& jb, const Span& sp) {
    KeyWalk<MASKED> w;
    KeyTile kt;
    int n = 0;
    while (w.next(jb, sp, kt)) n++;
    return n;
}

// ------------------------------------------------------------------------------------------ MMA
// S (128 x 128 f32, TMEM) = Q (128 rows, K-major, 128-byte swizzle) . K^T (128 keys, same layout):
// eight K=16 slices along the head dim.  Slice s sits 32 bytes further inside a 64-column panel,
// slices 4-7 in the second panel; the descriptor's address field counts 16-byte units.
FV_DEV void scores_mma(uint32_t tS, uint32_t q_smem, uint32_t k_smem) {
    constexpr uint32_t idesc = umma_idesc_bf16(kRowTile, kKeyTile, 0);
    const uint64_t qd = umma_desc_sw128(q_smem, 16, 1024), kd = umma_desc_sw128(k_smem, 16, 1024);
#pragma unroll
    for (int s = 0; s < 8; s++) {
        const uint64_t step = (uint64_t)((s & 3) * 2 + (s >> 2) * (int)(kPanelBytes >> 4));
        umma_ss(tS, qd + step, kd + step, idesc, s > 0 ? 1u : 0u);
    }
}
// O (128 x 128 f32, TMEM) (+)= P . V over the K=16 key slices named in SLICES (bit s = keys 16 s .. 16 s + 15).
// P comes from TMEM: slice s at column 64 (s / 4) + 8 (s % 4) of the row tile's score block.  V is
// MN-major in shared memory: 64-column panels 16 KB apart, 8-key groups 1024 bytes apart.
template <uint32_t SLICES>
FV_DEV void output_mma(uint32_t tO, uint32_t tS, uint32_t v_smem, bool fresh) {
    constexpr uint32_t idesc = umma_idesc_bf16(kRowTile, kD, 1);
    const uint64_t vd = umma_desc_sw128(v_smem, kPanelBytes, 1024);
    uint32_t acc = fresh ? 0u : 1u;
#pragma unroll
    for (int s = 0; s < 8; s++) {
        if (((SLICES >> s) & 1u) == 0u) continue;
        umma_ts(tO, tS + 64u * (uint32_t)(s >> 2) + 8u * (uint32_t)(s & 3), vd + (uint64_t)(s * 128), idesc, acc);
        acc = 1u;
    }
}

// -------------------------------------------------------------------------------------- softmax
// 2^(u * sl2 + noff) for columns C0 .. C0 + 31 of this thread's half row: packed bf16 pairs into
// pw[C0 / 2 .. C0 / 2 + 15], returns the f32 sum.  POLY: every fourth pair on the FMA pipe
// (fvp::ex2_poly_x2) instead of MUFU; only for tiles without masked columns, because the
// polynomial never returns an exact zero.
template <int C0, bool POLY>
FV_DEV float exp_chunk(const uint32_t (&u)[64], uint32_t (&pw)[32], float sl2, float noff) {
    uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
    const uint64_t s2 = pack_f32x2(sl2, sl2), nf = pack_f32x2(noff, noff);
#pragma unroll
    for (int w = 0; w < 16; w++) {
        const int c = C0 + 2 * w;
        float t0, t1, p0, p1;
        unpack_f32x2(fma_f32x2(pack_f32x2(as_f(u[c]), as_f(u[c + 1])), s2, nf), t0, t1);
        if (POLY && (w & 3) == 3) {
            ex2_poly_x2(t0, t1, p0, p1);
        } else {
            p0 = ex2(t0);
            p1 = ex2(t1);
        }
        const uint64_t pp = pack_f32x2(p0, p1);
        if (w & 1) acc1 = add_f32x2(acc1, pp);
        else acc0 = add_f32x2(acc0, pp);
        pw[C0 / 2 + w] = pack_bf16x2(p0, p1);
    }
    float a, b, c, d;
    unpack_f32x2(acc0, a, b);
    unpack_f32x2(acc1, c, d);
    return (a + b) + (c + d);
}

FV_DEV float max64(const uint32_t (&u)[64]) {
    float x0 = max3(as_f(u[0]), as_f(u[1]), as_f(u[2])), x1 = max3(as_f(u[3]), as_f(u[4]), as_f(u[5]));
    float x2 = max3(as_f(u[6]), as_f(u[7]), as_f(u[8])), x3 = max3(as_f(u[9]), as_f(u[10]), as_f(u[11]));
#pragma unroll
    for (int c = 12; c < 60; c += 8) {
        x0 = max3(x0, as_f(u[c]), as_f(u[c + 1]));
        x1 = max3(x1, as_f(u[c + 2]), as_f(u[c + 3]));
        x2 = max3(x2, as_f(u[c + 4]), as_f(u[c + 5]));
        x3 = max3(x3, as_f(u[c + 6]), as_f(u[c + 7]));
    }
    x0 = max3(x0, as_f(u[60]), as_f(u[61]));
    x1 = max3(x1, as_f(u[62]), as_f(u[63]));
    return fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
}

// The smallest bf16 at or above x, as the 16 high bits of its f32 pattern (-inf stays -inf).
FV_DEV uint16_t bf16_ceil(float x) {
    uint32_t b = as_u(x);
    if (x > 0.f && (b & 0xffffu)) b += 0x10000u;  // positive: truncation rounds down, step up
    return (uint16_t)(b >> 16);                    // negative: truncation already rounds toward zero, i.e. up
}
FV_DEV float bf16_bits_to_f(uint16_t h) { return as_f((uint32_t)h << 16); }

// Bounded wait on phase `parity` of a CTA barrier.  What it needs to give up cleanly (abort flag in
// shared memory, status word and cycle budget in the kernel's parameters) is fetched on the slow path
// only, so a role keeps no wait state in registers.  False after a timeout, or when another thread of
// the CTA has given up.
struct Waiter {
    const Job& jb;
    uint32_t sbase;
    int role;
    FV_DEV bool operator()(uint32_t bar, uint32_t parity) const {
        if (mbar_try(bar, parity)) return true;
        const long long t0 = clock64();
        uint32_t n = 0;
        while (!mbar_try(bar, parity)) {
            if (((++n) & 63u) == 0u) {
                uint32_t gone;
                asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(gone) : "r"(sbase + Smem::abort_flag) : "memory");
                if (gone) return false;
                if (clock64() - t0 > jb.wait_cycles) {
                    asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(sbase + Smem::abort_flag), "r"(1u) : "memory");
                    atomicCAS(jb.status, FV_ST_OK, FV_ST_TIMEOUT_BASE + role);
                    return false;
                }
            }
        }
        return true;
    }
};

FV_DEV void sts_u16(uint32_t addr, uint16_t v) {
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
FV_DEV uint16_t lds_u16(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr) : "memory");
    return v;
}

// One phase of the 64-thread barrier of a row's two warps.
FV_DEV bool pair_sync(uint32_t bar, uint32_t& count, const Waiter& wait) {
    mbar_arrive(bar);
    const bool ok = wait(bar, count & 1u);
    count++;
    return ok;
}

// 32 columns of one output row: O / l (+ the earlier pass' share), to bf16 or f32.
FV_DEV void store_cols32(const Job& jb, const uint32_t (&o)[32], float inv, float prev_w, const float* prev_row,
                         void* out_row) {
    float f[32];
#pragma unroll
    for (int c = 0; c < 32; c++) f[c] = as_f(o[c]) * inv;
    if (prev_row) {
        const float4* pr = reinterpret_cast<const float4*>(prev_row);
#pragma unroll
        for (int c = 0; c < 8; c++) {
            const float4 t = pr[c];
            f[4 * c] = fmaf(t.x, prev_w, f[4 * c]);
            f[4 * c + 1] = fmaf(t.y, prev_w, f[4 * c + 1]);
            f[4 * c + 2] = fmaf(t.z, prev_w, f[4 * c + 2]);
            f[4 * c + 3] = fmaf(t.w, prev_w, f[4 * c + 3]);
        }
    }
    if (jb.out_is_bf16) {
        uint4* dst = reinterpret_cast<uint4*>(out_row);
#pragma unroll
        for (int c = 0; c < 4; c++)
            dst[c] = make_uint4(pack_bf16x2(f[8 * c], f[8 * c + 1]), pack_bf16x2(f[8 * c + 2], f[8 * c + 3]),
                                pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), pack_bf16x2(f[8 * c + 6], f[8 * c + 7]));
    } else {
        float4* dst = reinterpret_cast<float4*>(out_row);
#pragma unroll
        for (int c = 0; c < 8; c++) dst[c] = make_float4(f[4 * c], f[4 * c + 1], f[4 * c + 2], f[4 * c + 3]);
    }
}

template <bool MASKED>
FV_DEV void softmax_warp(const Job& jb, uint32_t sbase, uint32_t tmem, int warp, int lane,
                         const Waiter& wait) {
    const int tile = warp >> 3, half = (warp >> 2) & 1, quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lanes = tmem + ((uint32_t)(quad * 32) << 16);
    const uint32_t tS = lanes + 256u * (uint32_t)tile + 64u * (uint32_t)half;          // this thread's 64 score columns
    const uint32_t tO = tS + 128u;                                                      // its 64 output columns
    const uint32_t bt = sbase + 8u * (uint32_t)tile;  // + Smem::{s_ready, p_early, p_ready, o_ready}: this row tile's barriers
    const uint32_t b_pair = sbase + Smem::pair + 8u * (uint32_t)(tile * 4 + quad);
    // exchange words of this row: u16 [parity 2] 512 bytes apart; the other half's are 256 bytes away
    const uint32_t mine = sbase + Smem::xch + 2u * (uint32_t)(tile * 512 + half * 128 + row);
    const uint32_t theirs = sbase + Smem::xch + 2u * (uint32_t)(tile * 512 + (1 - half) * 128 + row);
    const float sl2 = jb.sl2;
    uint32_t s_count = 0, o_count = 0, x_count = 0;

    for (int i = (int)blockIdx.x; i < jb.items; i += (int)gridDim.x) {
        const Item it = item_at(jb, i);
        const int qr = it.q0 + kRowTile * tile + row;  // this thread's row inside the plane
        const Span cta_span = span_of<MASKED>(jb, global_row(jb, it.q0), global_row(jb, min(it.q0 + kItemRows, jb.sq) - 1));
        const Span row_span = span_of<MASKED>(jb, global_row(jb, qr), global_row(jb, qr));
        float m = neg_inf(), l = 0.f;
        int seen = 0;
        KeyWalk<MASKED> walk;
        KeyTile kt;
        while (walk.next(jb, cta_span, kt)) {
            // (warp-uniform outcomes: the TMEM instructions below are warp-collective)
            if (!__all_sync(kFullWarp, wait(bt + Smem::s_ready, s_count & 1u))) return;
            s_count++;
            tc_fence_after();
            uint32_t u[64];
            tmem_ld32_at<0>(tS, u);
            tmem_ld32_at<32>(tS + 32u, u);
            tmem_ld_wait();
            tmem_pin(u);

            // columns of this half the row may not see become -inf
            const int kb = kt.k0 + 64 * half;
            const int nv = min(max(kt.valid - 64 * half, 0), 64);
            bool whole;
            if constexpr (MASKED) {
                const int c_lo = row_span.lo - kb, c_hi = min(row_span.hi - kb, nv), c_sink = min(row_span.sink - kb, nv);
                whole = (c_lo <= 0 && c_hi >= 64) || c_sink >= 64;
                if (!whole) {
#pragma unroll
                    for (int c = 0; c < 64; c++) {
                        const bool vis = (c >= c_lo && c < c_hi) || c < c_sink;
                        u[c] = vis ? u[c] : as_u(neg_inf());
                    }
                }
            } else {
                whole = nv == 64;
                if (!whole) {
#pragma unroll
                    for (int c = 0; c < 64; c++) u[c] = c < nv ? u[c] : as_u(neg_inf());
                }
            }

            // the two halves of the row agree on the tile's maximum
            const uint16_t mine_up = bf16_ceil(max64(u));
            const uint32_t par = x_count & 1u;
            sts_u16(mine + 512u * par, mine_up);
            if (!__all_sync(kFullWarp, pair_sync(b_pair, x_count, wait))) return;
            const float cand = fmaxf(bf16_bits_to_f(mine_up), bf16_bits_to_f(lds_u16(theirs + 512u * par))) * sl2;
            const bool grow = cand > m + kSlackLog2;
            float a = 1.f;
            if (grow) {
                a = ex2(m - cand);
                m = cand;
                l *= a;
            }
            // O holds P.V of the earlier tiles of the item (those MMAs were issued before the one that
            // produced this S, and S is complete): rescale this thread's 64 columns when a reference moved.
            if (seen > 0 && __any_sync(kFullWarp, grow)) {
#pragma unroll 1
                for (int q = 0; q < 2; q++) {
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
            uint32_t pw[32];
            float sum;
            // (warp-uniform choice: the TMEM stores are warp-collective)
            const bool poly = __all_sync(kFullWarp, whole);
            sum = poly ? exp_chunk<0, true>(u, pw, sl2, noff) : exp_chunk<0, false>(u, pw, sl2, noff);
            tmem_st16_at<0>(tS, pw);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bt + Smem::p_early);
            sum += poly ? exp_chunk<32, true>(u, pw, sl2, noff) : exp_chunk<32, false>(u, pw, sl2, noff);
            tmem_st16_at<16>(tS + 16u, pw);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(bt + Smem::p_ready);
            l += sum;
            seen++;
        }

        // ------------------------------------------------------------------------- the item's output
        if (seen > 0) {
            if (!__all_sync(kFullWarp, wait(bt + Smem::o_ready, o_count & 1u))) return;
            o_count++;
            tc_fence_after();
        }
        // Row sum = this half's + the other half's.  First phase: the partner has read this item's last
        // maximum out of the exchange words; second: both sums are written; third: both are read.
        if (!__all_sync(kFullWarp, pair_sync(b_pair, x_count, wait))) return;
        const uint32_t lbits = as_u(l);
        sts_u16(mine, (uint16_t)(lbits & 0xffffu));
        sts_u16(mine + 512u, (uint16_t)(lbits >> 16));
        if (!__all_sync(kFullWarp, pair_sync(b_pair, x_count, wait))) return;
        const float l_other = as_f((uint32_t)lds_u16(theirs) | ((uint32_t)lds_u16(theirs + 512u) << 16));
        if (!__all_sync(kFullWarp, pair_sync(b_pair, x_count, wait))) return;
        const float lsum = l + l_other;

        const bool live = qr < jb.sq;  // rows past sq only take part in the warp-collective TMEM loads
        float inv = lsum > 0.f ? 1.f / lsum : 0.f;
        const float lse = lsum > 0.f ? m + log2f(lsum) : neg_inf();
        const size_t rowi = (size_t)it.plane * jb.sq + (live ? qr : 0);
        float prev_w = 0.f;
        if (live) {
            if (jb.prev_o) {
                const float pl = jb.prev_lse[rowi];
                const float top = fmaxf(lse, pl);
                float lse_all = neg_inf();
                if (top != neg_inf()) {
                    const float wn = exp2f(lse - top), wp = exp2f(pl - top);
                    const float den = 1.f / (wn + wp);
                    inv *= wn * den;
                    prev_w = wp * den;
                    lse_all = top + log2f(wn + wp);
                }
                if (jb.lse_out && half == 0) jb.lse_out[rowi] = lse_all;
            } else if (jb.lse_out && half == 0) {
                jb.lse_out[rowi] = lse;
            }
        }
        size_t out_el = rowi * kD;  // BHSD element offset of the row (also the earlier pass' layout)
        const size_t prev_el = out_el;
        if (jb.out_heads > 0) {
            const int bb = it.plane / jb.out_heads, hh = it.plane - bb * jb.out_heads;
            out_el = (((size_t)bb * jb.sq + (live ? qr : 0)) * jb.out_heads + hh) * kD;
        }
#pragma unroll 1
        for (int q = 0; q < 2; q++) {
            uint32_t o[32];
            if (seen > 0) {  // warp-uniform
                tmem_ld32_issue(tO + 32u * q, o);
                tmem_ld_wait();
                tmem_pin(o);
            } else {
#pragma unroll
                for (int c = 0; c < 32; c++) o[c] = 0u;
            }
            if (!live) continue;
            const int col = 64 * half + 32 * q;
            void* dst = jb.out_is_bf16 ? (void*)(reinterpret_cast<unsigned short*>(jb.out) + out_el + col)
                                       : (void*)(reinterpret_cast<float*>(jb.out) + out_el + col);
            store_cols32(jb, o, inv, prev_w, jb.prev_o ? jb.prev_o + prev_el + col : nullptr, dst);
        }
        // The next item's first P.V overwrites O.  The issuer issues it only after all 256 threads of the
        // row tile have arrived at p_ready for that item's first key tile, and a thread gets there only
        // after its loads above have completed.
    }
}

// --------------------------------------------------------------------------------------- loader
template <bool MASKED>
FV_DEV void loader_thread(const CUtensorMap* mq, const CUtensorMap* mk, const CUtensorMap* mv, const Job& jb,
                          uint32_t sbase, const Waiter& wait) {
    uint32_t qn = 0, kvn = 0;  // Q tiles and K/V tiles loaded so far
    tma_prefetch_desc(mq);
    tma_prefetch_desc(mk);
    tma_prefetch_desc(mv);
    auto load_q = [&](int item, int tile) -> bool {
        const Item it = item_at(jb, item);
        const uint32_t slot = qn % kQSlots, use = qn / kQSlots;
        if (use > 0 && !wait(sbase + Smem::q_free + 8u * slot, (use - 1u) & 1u)) return false;
        const uint32_t dst = sbase + Smem::q + slot * kSlotBytes, bar = sbase + Smem::q_full + 8u * slot;
        const int plane = jb.q_div > 1 ? it.plane / jb.q_div : it.plane;
        const int r0 = it.q0 + kRowTile * tile;  // rows past sq read as zeros
        mbar_expect_tx(bar, kSlotBytes);
        tma_load4(dst, mq, bar, 0, r0, plane, 0);
        tma_load4(dst + kPanelBytes, mq, bar, 64, r0, plane, 0);
        qn++;
        return true;
    };
    auto load_kv = [&](const CUtensorMap* map, const KeyTile& kt, int plane) -> bool {
        const uint32_t slot = kvn % kKvSlots, use = kvn / kKvSlots;
        if (use > 0 && !wait(sbase + Smem::kv_free + 8u * slot, (use - 1u) & 1u)) return false;
        const uint32_t dst = sbase + Smem::kv + slot * kSlotBytes, bar = sbase + Smem::kv_full + 8u * slot;
        mbar_expect_tx(bar, kSlotBytes);
        tma_load4(dst, map, bar, 0, kt.t * kKeyTile, plane, kt.seg);
        tma_load4(dst + kPanelBytes, map, bar, 64, kt.t * kKeyTile, plane, kt.seg);
        kvn++;
        return true;
    };

    int i = (int)blockIdx.x;
    bool ok = true;
    if (i < jb.items) ok = load_q(i, 0) && load_q(i, 1);
    for (; ok && i < jb.items; i += (int)gridDim.x) {
        const int nxt = i + (int)gridDim.x;
        // Row tile A of the next item goes into the slot the previous item's tile B left long ago.
        if (nxt < jb.items) ok = load_q(nxt, 0);
        const Item it = item_at(jb, i);
        const Span sp = span_of<MASKED>(jb, global_row(jb, it.q0), global_row(jb, min(it.q0 + kItemRows, jb.sq) - 1));
        KeyWalk<MASKED> walk;
        KeyTile kt;
        while (ok && walk.next(jb, sp, kt)) ok = load_kv(mk, kt, it.plane) && load_kv(mv, kt, it.plane);
        // Tile B of the next item takes the slot of this item's tile A, free after its last Q.K^T.
        if (ok && nxt < jb.items) ok = load_q(nxt, 1);
    }
    // Copies in flight must land before the CTA's shared memory goes away.  After a clean run the
    // issuer has waited on every one of these phases already and the loops fall straight through.
    for (uint32_t s = 0; s < (uint32_t)kQSlots && s < qn; s++) {
        const uint32_t last = ((qn - 1u - s) / kQSlots) * kQSlots + s;  // last load that used slot s
        mbar_drain(sbase + Smem::q_full + 8u * s, (last / kQSlots) & 1u);
    }
    for (uint32_t s = 0; s < (uint32_t)kKvSlots && s < kvn; s++) {
        const uint32_t last = ((kvn - 1u - s) / kKvSlots) * kKvSlots + s;
        mbar_drain(sbase + Smem::kv_full + 8u * s, (last / kKvSlots) & 1u);
    }
}

// --------------------------------------------------------------------------------------- issuer
// P_t(j) . V(j) into O_t.  The first product of an item overwrites O, which the softmax threads of
// the previous item may still be reading until every one of them has stored the whole of this tile's
// P: that product waits for p_ready first; later ones start on the early half.
FV_DEV bool issue_output(uint32_t sbase, int t, uint32_t tmem, uint32_t v_smem, bool fresh, uint32_t& p_count,
                         const Waiter& wait) {
    const uint32_t tS = tmem + 256u * (uint32_t)t, tO = tS + 128u;
    const uint32_t b_pe = sbase + Smem::p_early + 8u * t, b_pr = sbase + Smem::p_ready + 8u * t;
    const uint32_t par = p_count & 1u;
    p_count++;
    if (fresh) {
        if (!wait(b_pe, par) || !wait(b_pr, par)) return false;
        tc_fence_after();
        output_mma<0xffu>(tO, tS, v_smem, true);
        return true;
    }
    if (!wait(b_pe, par)) return false;
    tc_fence_after();
    output_mma<0x33u>(tO, tS, v_smem, false);  // keys 0-31 and 64-95
    if (!wait(b_pr, par)) return false;
    tc_fence_after();
    output_mma<0xccu>(tO, tS, v_smem, false);  // keys 32-63 and 96-127
    return true;
}

template <bool MASKED>
FV_DEV void issuer_thread(const Job& jb, uint32_t sbase, uint32_t tmem, const Waiter& wait) {
    uint32_t qn = 0, kvn = 0;
    uint32_t p_count[2] = {0u, 0u};
    bool ok = true;
    for (int i = (int)blockIdx.x; ok && i < jb.items; i += (int)gridDim.x) {
        const Item it = item_at(jb, i);
        const Span sp = span_of<MASKED>(jb, global_row(jb, it.q0), global_row(jb, min(it.q0 + kItemRows, jb.sq) - 1));
        const int n = count_tiles<MASKED>(jb, sp);
        uint32_t q_slot[2], q_smem[2], q_par[2];
#pragma unroll
        for (int t = 0; t < 2; t++) {
            q_slot[t] = (qn + t) % kQSlots;
            q_par[t] = ((qn + t) / kQSlots) & 1u;
            q_smem[t] = sbase + Smem::q + q_slot[t] * kSlotBytes;
        }
        qn += 2;
        if (n == 0) {
            // No key of any segment is visible to these rows.  The Q tiles were loaded all the same: let
            // them land before their slots are handed back.
#pragma unroll
            for (int t = 0; t < 2; t++) {
                if (ok && !wait(sbase + Smem::q_full + 8u * q_slot[t], q_par[t])) ok = false;
                if (ok) mbar_arrive(sbase + Smem::q_free + 8u * q_slot[t]);
            }
            continue;
        }
        for (int j = 0; ok && j < n; j++) {
            const uint32_t ik = kvn + 2u * (uint32_t)j, k_slot = ik % kKvSlots;
            const uint32_t k_smem = sbase + Smem::kv + k_slot * kSlotBytes;
            uint32_t v_slot = 0, v_smem = 0;
            if (j > 0) {  // V(j-1) was loaded before K(j): the products that need it go first
                const uint32_t iv = ik - 1u;
                v_slot = iv % kKvSlots;
                if (!wait(sbase + Smem::kv_full + 8u * v_slot, (iv / kKvSlots) & 1u)) { ok = false; break; }
                v_smem = sbase + Smem::kv + v_slot * kSlotBytes;
                tc_fence_after();
            }
#pragma unroll
            for (int t = 0; t < 2; t++) {
                if (j > 0 && ok) ok = issue_output(sbase, t, tmem, v_smem, j == 1, p_count[t], wait);
                if (t == 0 && ok) {
                    if (!wait(sbase + Smem::kv_full + 8u * k_slot, (ik / kKvSlots) & 1u)) ok = false;
                    tc_fence_after();
                }
                // (tile B of an item is loaded late, see loader_thread: it is waited for where it is first used)
                if (j == 0 && ok && !wait(sbase + Smem::q_full + 8u * q_slot[t], q_par[t])) ok = false;
                if (!ok) break;
                if (j == 0) tc_fence_after();
                scores_mma(tmem + 256u * (uint32_t)t, q_smem[t], k_smem);
                umma_commit(sbase + Smem::s_ready + 8u * t);
                if (j == n - 1) umma_commit(sbase + Smem::q_free + 8u * q_slot[t]);
            }
            if (!ok) break;
            if (j > 0) umma_commit(sbase + Smem::kv_free + 8u * v_slot);
            umma_commit(sbase + Smem::kv_free + 8u * k_slot);
        }
        if (!ok) break;
        {   // the last key tile's P.V
            const uint32_t iv = kvn + 2u * (uint32_t)n - 1u, v_slot = iv % kKvSlots;
            if (!wait(sbase + Smem::kv_full + 8u * v_slot, (iv / kKvSlots) & 1u)) break;
            tc_fence_after();
            const uint32_t v_smem = sbase + Smem::kv + v_slot * kSlotBytes;
#pragma unroll
            for (int t = 0; t < 2; t++) {
                if (ok) ok = issue_output(sbase, t, tmem, v_smem, n == 1, p_count[t], wait);
                if (ok) umma_commit(sbase + Smem::o_ready + 8u * t);
            }
            if (!ok) break;
            umma_commit(sbase + Smem::kv_free + 8u * v_slot);
        }
        kvn += 2u * (uint32_t)n;
    }
    // Nothing this thread issued may still be running when TMEM is freed.
    umma_commit(sbase + Smem::drain);
    mbar_drain(sbase + Smem::drain, 0);
}

// ----------------------------------------------------------------------------------- the kernel
template <bool MASKED>
FV_DEV void attn_persistent(const CUtensorMap* mq, const CUtensorMap* mk, const CUtensorMap* mv, const Job& jb,
                            unsigned char* smem) {
    const uint32_t sbase = smem_u32(smem);
    const int warp = (int)(threadIdx.x >> 5), lane = (int)(threadIdx.x & 31);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + Smem::abort_flag);
    volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem + Smem::tmem_slot);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kQSlots; s++) {
            mbar_init(sbase + Smem::q_full + 8u * s, 1);
            mbar_init(sbase + Smem::q_free + 8u * s, 1);
        }
        for (int s = 0; s < kKvSlots; s++) {
            mbar_init(sbase + Smem::kv_full + 8u * s, 1);
            mbar_init(sbase + Smem::kv_free + 8u * s, 1);
        }
        for (int t = 0; t < 2; t++) {
            mbar_init(sbase + Smem::s_ready + 8u * t, 1);
            mbar_init(sbase + Smem::p_early + 8u * t, 256);
            mbar_init(sbase + Smem::p_ready + 8u * t, 256);
            mbar_init(sbase + Smem::o_ready + 8u * t, 1);
        }
        for (int p = 0; p < 8; p++) mbar_init(sbase + Smem::pair + 8u * p, 64);
        mbar_init(sbase + Smem::drain, 1);
        // A CTA that starts after another one gave up does nothing.
        int bad = (*(volatile int*)jb.status != FV_ST_OK) ? 1 : 0;
        if (sbase & 1023u) {
            atomicCAS(jb.status, FV_ST_OK, FV_ST_BAD_SMEM);
            bad = 1;
        }
        *abort_flag = bad;
        mbar_init_fence();
    }
    __syncthreads();
    if (*abort_flag) return;  // CTA-uniform
    if (warp == kIssuerWarp) tmem_alloc(sbase + Smem::tmem_slot, 512);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp < kSoftmaxWarps) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 104;" ::: "memory");
        softmax_warp<MASKED>(jb, sbase, tmem, warp, lane, Waiter{jb, sbase, 3});
    } else {
        // (one setmaxnreg for the whole warpgroup: warps 16-19 execute this very instruction together)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 64;" ::: "memory");
        if (lane == 0) {
            if (warp == kLoaderWarp) loader_thread<MASKED>(mq, mk, mv, jb, sbase, Waiter{jb, sbase, 1});
            else if (warp == kIssuerWarp) issuer_thread<MASKED>(jb, sbase, tmem, Waiter{jb, sbase, 2});
        }
        __syncwarp();
    }
    // Every TMEM access of every thread is complete: the allocation may go.
    tc_fence_before();
    __syncthreads();
    if (warp == kIssuerWarp) {
        tc_fence_after();
        tmem_dealloc(tmem, 512);
    }
}

#endif  // sm_100a / host pass

}  // namespace fvattn

// Persistent flash-attention forward for head dim 128 on sm_100a.
//
// Operand convention of the launcher it replaces (crates/fastvideo-cudarc/src/rt/attn_dc.rs:213-273,
// dense_fwd, and the block-causal launcher crates/fastvideo-cudarc/src/rt/attn.rs:647-730): bf16
// [planes, s, 128] in, bf16 or f32 [planes, sq, 128] out, scores scaled by sl2 = scale * log2 e.
//
// Shape of the kernel
// -------------------
// * One CTA per SM for the whole launch.  Work items (256 query rows of one plane = two 128-row
//   accumulator tiles, "A" and "B") are dealt in snake order: in round r CTA c takes item r G + c, in the
//   next one item (r + 1) G + (G - 1 - c).  Under a mask the items are ordered heaviest first.
// * 12 warps = three warpgroups.  The launch gives every thread 168 registers; the two softmax
//   warpgroups then take 216 each and the third drops to 72 (256 x 216 + 128 x 72 = 384 x 168):
//     warps 0-7    softmax: warp w serves row tile w / 4, TMEM lanes 32 (w % 4) .. + 31 (thread =
//                  TMEM lane = query row, the only mapping the 32x32b TMEM load offers).
//     warp 8       loader: one thread issues every TMA copy (Q ring of 3 x 32 KB; K/V ring of 4 x 32 KB
//                  filled in PAIRS [V(j-1) | K(j)], one barrier per pair) and runs one item ahead with
//                  the Q tiles.
//     warp 9       issuer: one thread issues every tcgen05.mma; the warp owns the TMEM allocation.
//     warps 10-11  idle (they make the third warpgroup whole).
// * TMEM (512 columns): scores S_A, S_B (128 f32 columns each), then the output accumulators O_A,
//   O_B.  The bf16 probabilities P overwrite S from its column 0 on (64 columns), always behind the
//   columns still to be read.
// * Per key tile j the issuer runs, for t = A then B:  O_t += P_t(j-1) . V(j-1);  S_t = Q_t . K(j)^T,
//   strictly in order, so one row tile's softmax runs under the other's MMAs and the two tiles stay half a
//   period apart (the MUFU pipe of a scheduler then serves one tile's exponentials at a time).  Per step the
//   issuer waits three times (the K/V pair, P_A, P_B) and commits four times: every wait and commit is a
//   point where it can stall while the tensor pipe's short queue runs dry, and halving their number (pairs
//   instead of single tiles, P handed over whole instead of in two parts) was worth 9 % and 7 % of the
//   step.  SM-clock stamps of one CTA's roles (a bring-up build, -DFV_ATT_TRACE) are how this was found.
// * STREAMING softmax without a maximum pass.  Base-2 domain, lazy reference m per row: P = 2^(s -
//   m) is evaluated straight away against the reference the row already has, 32 columns at a time as
//   they come out of TMEM (the next chunk's load in flight), a quarter of the exponentials on the FMA
//   pipe, and the row's sum of P is the proof that this was safe: every P is positive, so sum(P) <= 2^40
//   implies max(P) <= 2^40, far inside what bf16 P and f32 accumulators hold, and a reference that lags
//   the true maximum by any amount cancels exactly when O is divided by the row sum.  A row without a
//   reference (the first tile of an item) takes the maximum of its first 32 scores as one.  Only when a sum
//   exceeds the guard, or a mask or a segment's end cuts the tile, does the warp take the exact path:
//   nothing of the tile has been stored, so it reads S again, takes the row maxima, moves the references,
//   rescales O and the row sums, evaluates P again.  On N(0,1) inputs without a mask the exact path runs on
//   ragged last tiles and nowhere else.
// * The item's output (write_item) is on the critical path of the next item -- the same warps run its
//   first softmax -- and with few key tiles per item (cross-attention: 4) it is a third of the item.  It
//   runs out of line (its registers are not the hot loop's), loads O from TMEM in two alternating
//   32-column buffers, transposes 16-byte pieces between neighbouring lanes so that a warp's store covers
//   whole 64- or 128-byte runs of 8 or 4 rows instead of 16 bytes of 32 rows, and the softmax warp looks
//   up its next item before it waits for the last product, not after the output.  Together 12 % of the
//   item at 4 key tiles (20 300 -> 17 800 cycles), nothing at 256 and more.
// * Every wait is bounded: a role that gives up records a code in the status word, raises the CTA's
//   abort flag, and every role falls through to the common exit, where copies in flight are awaited,
//   the issuer's last MMA is awaited and TMEM is freed.  No trap, no endless spin.
#pragma once
#include <cuda.h>
#include "fv_ptx.cuh"

// Build-time tuning (every setting computes the same function):
//   FV_ATT_POLY     every FV_ATT_POLY-th pair of an unmasked tile's exponentials is evaluated on the FMA pipe
//                   instead of MUFU (0 = none, 4 = a quarter, 8 = an eighth, 2 = a half).  Both tiles' softmax
//                   warps share one MUFU pipe per scheduler (4 results per cycle), which at 128 x 128
//                   exponentials per tile is exactly as long as the tile's two MMAs: moving a share of them
//                   to the FMA pipe, evenly interleaved, is what lets the two overlap.
//   FV_ATT_EARLY    keys of a tile whose P is handed to the issuer first (64 or 96), the rest follows; 128: P is
//                   handed over whole (one wait and no pv_early commit per tile for the issuer)
//   FV_ATT_SPLIT    TMEM map: 1 = S_A S_B O_A O_B, 0 = S_A O_A S_B O_B (no measurable difference)
//   FV_ATT_WAIT_HINT  > 0: every barrier wait passes this many nanoseconds to mbarrier.try_wait as the longest
//                   suspension before the thread looks again (0: the hardware's default)
//   FV_ATT_BACKOFF  nanoseconds a waiting softmax thread sleeps between two probes of its barrier (0 = none);
//                   FV_ATT_BACKOFF_LOADER the same for the loader thread
#ifndef FV_ATT_POLY
#define FV_ATT_POLY 4
#endif
#ifndef FV_ATT_EARLY
#define FV_ATT_EARLY 128
#endif
#ifndef FV_ATT_SPLIT
#define FV_ATT_SPLIT 1
#endif
#ifndef FV_ATT_WAIT_HINT
#define FV_ATT_WAIT_HINT 0
#endif
#ifndef FV_ATT_BACKOFF
#define FV_ATT_BACKOFF 0
#endif
#ifndef FV_ATT_BACKOFF_LOADER
#define FV_ATT_BACKOFF_LOADER 0
#endif

#define FV_ST_BAD_SMEM 90  // dynamic shared memory is not 1024-byte aligned (the swizzled tiles need it)

namespace fvattn {

constexpr int kD = 128;
constexpr int kKeyTile = 128;   // keys per score tile: N of Q.K^T, K extent of P.V
constexpr int kRowTile = 128;   // query rows per accumulator: M of both products
constexpr int kItemRows = 256;  // one work item = row tiles A and B
constexpr int kWarps = 12;
constexpr int kThreads = kWarps * 32;
constexpr int kSoftmaxWarps = 8;
constexpr int kLoaderWarp = 8;
constexpr int kIssuerWarp = 9;
constexpr int kQSlots = 3;
constexpr int kKvSlots = 4;     // 32 KB tiles; they are filled and freed in PAIRS [V(j-1) | K(j)]: one barrier each way per step
constexpr int kKvPairs = kKvSlots / 2;
constexpr uint32_t kSlotBytes = 32768;   // 128 rows x 128 bf16: two 64-column swizzled panels
constexpr uint32_t kPanelBytes = 16384;
constexpr int kMaxSeg = 16;
constexpr float kGuard = 1099511627776.f;  // 2^40: a row sum of P above this sends the tile down the exact path
constexpr uint32_t kFullWarp = 0xffffffffu;
constexpr int kEarlyKeys = FV_ATT_EARLY;       // P of keys [0, kEarlyKeys) is stored and signalled first (p_early)
constexpr int kEarlyChunks = kEarlyKeys / 32;  // in 32-column chunks of S
static_assert(kEarlyKeys == 64 || kEarlyKeys == 96 || kEarlyKeys == 128, "FV_ATT_EARLY is 64, 96 or 128 (128: P handed over whole)");

// Shared-memory map, offsets from the (1024-byte aligned) start of dynamic shared memory.
struct Smem {
    static constexpr uint32_t q = 0;
    static constexpr uint32_t kv = q + kQSlots * kSlotBytes;
    static constexpr uint32_t q_full = kv + kKvSlots * kSlotBytes;  // mbarriers, 8 bytes each
    static constexpr uint32_t q_free = q_full + 8 * kQSlots;
    static constexpr uint32_t kv_full = q_free + 8 * kQSlots;
    static constexpr uint32_t kv_free = kv_full + 8 * kKvSlots;  // (kKvPairs of each are used)
    static constexpr uint32_t s_ready = kv_free + 8 * kKvSlots;  // [2] S_t complete (issuer -> softmax)
    static constexpr uint32_t p_early = s_ready + 16;            // [2] the early keys of P_t stored (softmax -> issuer)
    static constexpr uint32_t p_ready = p_early + 16;            // [2] all of P_t stored
    static constexpr uint32_t pv_early = p_ready + 16;           // [2] the product over the early keys has run (issuer -> softmax)
    static constexpr uint32_t o_ready = pv_early + 16;           // [2] O_t of the item complete
    static constexpr uint32_t drain = o_ready + 16;              // [2] everything an issuer thread issued has completed
    static constexpr uint32_t tmem_slot = drain + 16;
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
#ifdef FV_ATT_TRACE
    unsigned long long* trace;  // bring-up builds only: [3 roles][trace_steps][8] SM clock stamps of CTA 0
    int trace_steps;
#endif
};

// Bring-up instrumentation, compiled only with -DFV_ATT_TRACE (never in the shipped library): CTA 0's
// issuer (role 2) and lane 0 of the first softmax warp of each row tile (roles 0, 1) stamp the SM clock.
#ifdef FV_ATT_TRACE
#define FV_TR(jb, role, step, ev)                                                                       \
    do {                                                                                                \
        if (blockIdx.x == 0 && (jb).trace && (int)(step) < (jb).trace_steps)                            \
            (jb).trace[(((size_t)(role) * (jb).trace_steps) + (step)) * 8 + (ev)] = (unsigned long long)clock64(); \
    } while (0)
#else
#define FV_TR(jb, role, step, ev) do { } while (0)
#endif

#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL) || !defined(__CUDA_ARCH__)

using namespace fvp;

// TMEM columns of row tile t: its scores (the probabilities overwrite them from the first column on)
// and its output accumulator.
FV_DEV uint32_t tmem_scores(uint32_t t) { return FV_ATT_SPLIT ? 128u * t : 256u * t; }
FV_DEV uint32_t tmem_output(uint32_t t) { return FV_ATT_SPLIT ? 256u + 128u * t : 256u * t + 128u; }

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
// Work item number i.  Dense launches: plane-major, so the CTAs running at any one time share a few
// planes' K and V in L2.  Masked launches (jb.heavy_first): by falling cost, i.e. query block from the
// last to the first, every plane's copy of a block side by side.
FV_DEV Item item_at(const Job& jb, int i) {
    Item it;
    if (jb.heavy_first) {
        const int qb = jb.q_blocks - 1 - i / jb.planes;
        it.plane = i - (i / jb.planes) * jb.planes;
        it.q0 = qb * kItemRows;
    } else {
        it.plane = i / jb.q_blocks;
        it.q0 = (i - it.plane * jb.q_blocks) * kItemRows;
    }
    return it;
}
// The items of this CTA, in order: round r deals items r * grid .. r * grid + grid - 1, left to right
// in even rounds and right to left in odd ones.  With the items sorted by falling cost, a CTA that got
// the heaviest of one round gets the lightest of the next, and all CTAs end at about the same time.
struct Deal {
    int round = 0;
    FV_DEV int next(const Job& jb) {
        const int g = (int)gridDim.x, c = (int)blockIdx.x;
        const int i = round * g + (((round & 1) && jb.heavy_first) ? g - 1 - c : c);
        round++;
        return i < jb.items ? i : -1;
    }
    // (in an odd round of a masked launch the last, partial round is dealt from the right: the CTAs on the left,
    // which carried the heavier items of the round before, stay idle)
    FV_DEV int peek(const Job& jb) const {
        Deal d = *this;
        return d.next(jb);
    }
};

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
// The issuing thread is the pace-maker of the whole CTA: a tcgen05.mma of this size occupies the tensor
// pipe for 64 cycles, and one thread executing dependent integer instructions at one per four to six
// cycles falls behind as soon as an MMA costs it more than about ten instructions.  So every group of
// MMAs is ONE asm statement whose descriptors are the group's base descriptor plus a constant (in the
// 16-byte address field), two adds per MMA, and the thread keeps next to nothing in registers.
#define FV_MMA_SS "tcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
#define FV_MMA_TS "tcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
#define FV_QK_STEP(off) "add.s64 a, %1, " #off ";\n\tadd.s64 b, %2, " #off ";\n\t" FV_MMA_SS
#define FV_PV_STEP(col, off) "add.u32 t, %1, " #col ";\n\tadd.s64 b, %2, " #off ";\n\t" FV_MMA_TS

// S (128 x 128 f32, TMEM) = Q (128 rows, K-major, 128-byte swizzle) . K^T (128 keys, same layout):
// eight K=16 slices along the head dim.  Slice s sits 32 bytes (2 address units) further inside a
// 64-column panel, slices 4-7 in the second panel 16 KB (1024 units) on.
FV_DEV void scores_mma(uint32_t tS, uint64_t qd, uint64_t kd) {
    constexpr uint32_t idesc = umma_idesc_bf16(kRowTile, kKeyTile, 0);
    asm volatile(
        "{\n\t.reg .pred pt, pf;\n\t.reg .b64 a, b;\n\t"
        "setp.ne.b32 pf, %3, %3;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
        FV_QK_STEP(2) FV_QK_STEP(4) FV_QK_STEP(6) FV_QK_STEP(1024) FV_QK_STEP(1026) FV_QK_STEP(1028) FV_QK_STEP(1030)
        "}"
        ::"r"(tS), "l"(qd), "l"(kd), "r"(idesc)
        : "memory");
}
// O (128 x 128 f32, TMEM) (+)= P . V.  P comes from TMEM: key slice s (16 keys) at column 8 s of the
// row tile's score block.  V is MN-major in shared memory (64-column
// panels 16 KB apart, 8-key groups 1024 bytes apart): slice s starts 2 KB = 128 address units further.
// Two statements: keys [0, kEarlyKeys) (the first slice overwrites O when `fresh`) and the rest.
FV_DEV void output_mma_early(uint32_t tO, uint32_t tP, uint64_t vd, bool fresh) {
    constexpr uint32_t idesc = umma_idesc_bf16(kRowTile, kD, 1);
    asm volatile(
        "{\n\t.reg .pred pt, p0;\n\t.reg .b64 b;\n\t.reg .b32 t;\n\t"
        "setp.eq.b32 p0, %4, 0;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
        FV_PV_STEP(8, 128) FV_PV_STEP(16, 256) FV_PV_STEP(24, 384)
#if FV_ATT_EARLY >= 96
        FV_PV_STEP(32, 512) FV_PV_STEP(40, 640)
#endif
#if FV_ATT_EARLY == 128
        FV_PV_STEP(48, 768) FV_PV_STEP(56, 896)
#endif
        "}"
        ::"r"(tO), "r"(tP), "l"(vd), "r"(idesc), "r"(fresh ? 1u : 0u)
        : "memory");
}
FV_DEV void output_mma_late(uint32_t tO, uint32_t tP, uint64_t vd) {
    constexpr uint32_t idesc = umma_idesc_bf16(kRowTile, kD, 1);
    if (kEarlyKeys == 128) return;
    asm volatile(
        "{\n\t.reg .pred pt;\n\t.reg .b64 b;\n\t.reg .b32 t;\n\t"
        "setp.eq.b32 pt, %3, %3;\n\t"
#if FV_ATT_EARLY == 64
        FV_PV_STEP(32, 512) FV_PV_STEP(40, 640)
#endif
        FV_PV_STEP(48, 768) FV_PV_STEP(56, 896)
        "}"
        ::"r"(tO), "r"(tP), "l"(vd), "r"(idesc)
        : "memory");
}

// -------------------------------------------------------------------------------------- softmax
// Bounded wait on phase `parity` of a CTA barrier.  What it needs to give up cleanly (abort flag in
// shared memory, status word and cycle budget in the kernel's parameters) is fetched on the slow path
// only, so a role keeps no wait state in registers.  Every probe of a barrier is a shared-memory access
// that competes with the operand reads of the MMAs in flight -- a tight two-instruction spin in the ten
// waiting warps cost 13 % of the kernel -- so a waiter backs off between probes (FV_ATT_BACKOFF ns).
// False after a timeout, or when another thread of the CTA has given up.
struct Waiter {
    const Job& jb;
    uint32_t sbase;
    int role;
    FV_DEV bool probe(uint32_t bar, uint32_t parity) const {
#if FV_ATT_WAIT_HINT > 0
        return mbar_try_hint(bar, parity, FV_ATT_WAIT_HINT) != 0u;
#else
        return mbar_try(bar, parity) != 0u;
#endif
    }
    FV_DEV bool operator()(uint32_t bar, uint32_t parity) const {
        if (probe(bar, parity)) return true;
        const long long t0 = clock64();
        uint32_t n = 0;
        while (!probe(bar, parity)) {
            if (role == 1) {
                if (FV_ATT_BACKOFF_LOADER > 0) __nanosleep(FV_ATT_BACKOFF_LOADER);
            } else if (role == 3) {
                if (FV_ATT_BACKOFF > 0) __nanosleep(FV_ATT_BACKOFF);
            }
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

// One arrival for the whole warp: every lane has finished what the barrier publishes (TMEM stores
// followed by tcgen05.wait::st and fence::before_thread_sync), the warp meets, one lane arrives.
FV_DEV void warp_arrive(uint32_t bar, int lane) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
}

// 2^(u * sl2 + noff) for 32 score columns: packed bf16 pairs into pw[0 .. 15]; the f32 values are
// added into the two packed accumulators.  POLY: every FV_ATT_POLY-th pair goes through the FMA-pipe
// exponential (fvp::ex2_poly_x2) instead of MUFU; only for tiles without masked columns, because the
// polynomial never returns an exact zero.  The polynomial wraps around above 2^127 instead of giving
// inf, which the caller's sum guard could not see: the largest argument given to it is kept in `top`
// (one three-input max per pair) and checked with the sum.
template <bool POLY>
FV_DEV void exp32(const uint32_t (&u)[32], uint32_t* pw, uint64_t s2, uint64_t nf, uint64_t& acc0, uint64_t& acc1, float& top) {
#pragma unroll
    for (int w = 0; w < 16; w++) {
        float t0, t1, p0, p1;
        unpack_f32x2(fma_f32x2(pack_f32x2(as_f(u[2 * w]), as_f(u[2 * w + 1])), s2, nf), t0, t1);
        constexpr int kEvery = FV_ATT_POLY > 0 ? FV_ATT_POLY : 1;
        if (POLY && FV_ATT_POLY > 0 && (w % kEvery) == kEvery - 1) {
            top = max3(top, t0, t1);
            ex2_poly_x2(t0, t1, p0, p1);
        } else {
            p0 = ex2(t0);
            p1 = ex2(t1);
        }
        const uint64_t pp = pack_f32x2(p0, p1);
        if (w & 1) acc1 = add_f32x2(acc1, pp);
        else acc0 = add_f32x2(acc0, pp);
        pw[w] = pack_bf16x2(p0, p1);
    }
}

FV_DEV float max32(const uint32_t (&u)[32]) {
    float x0 = max3(as_f(u[0]), as_f(u[1]), as_f(u[2])), x1 = max3(as_f(u[3]), as_f(u[4]), as_f(u[5]));
    float x2 = max3(as_f(u[6]), as_f(u[7]), as_f(u[8])), x3 = max3(as_f(u[9]), as_f(u[10]), as_f(u[11]));
#pragma unroll
    for (int c = 12; c < 28; c += 8) {
        x0 = max3(x0, as_f(u[c]), as_f(u[c + 1]));
        x1 = max3(x1, as_f(u[c + 2]), as_f(u[c + 3]));
        x2 = max3(x2, as_f(u[c + 4]), as_f(u[c + 5]));
        x3 = max3(x3, as_f(u[c + 6]), as_f(u[c + 7]));
    }
    x0 = max3(x0, as_f(u[28]), as_f(u[29]));
    x1 = max3(x1, as_f(u[30]), as_f(u[31]));
    return fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
}

// Columns of one row of a key tile that the row may see: [lo, hi) U [0, sink), tile-relative.
struct Cols {
    int lo, hi, sink;
    bool whole;  // every one of the 128 columns is visible
    FV_DEV void hide(uint32_t (&x)[32], int c0) const {  // columns c0 .. c0 + 31: the invisible ones become -inf
        if (whole) return;
#pragma unroll
        for (int c = 0; c < 32; c++) {
            const bool vis = (c0 + c >= lo && c0 + c < hi) || c0 + c < sink;
            x[c] = vis ? x[c] : as_u(neg_inf());
        }
    }
};

// Sum of the four lanes of two packed accumulators; with POLY an argument the polynomial cannot take makes
// the sum infinite, so that the caller's guard sends the tile the careful way.
template <bool POLY>
FV_DEV float part_sum(uint64_t acc0, uint64_t acc1, float top) {
    float a, b, c, d;
    unpack_f32x2(acc0, a, b);
    unpack_f32x2(acc1, c, d);
    const float sum = (a + b) + (c + d);
    return (POLY && top > 120.f) ? __int_as_float(0x7f800000) : sum;
}
// One 32-column chunk of this thread's row of S: issue, and "landed" (every chunk issued so far is in registers).
FV_DEV void load_chunk(uint32_t tS, int chunk, uint32_t (&u)[32]) { tmem_ld32_issue(tS + 32u * (uint32_t)chunk, u); }
FV_DEV void land_chunk(uint32_t (&u)[32]) {
    tmem_ld_wait();
    tmem_pin(u);
}
// The stores of P issued so far are complete and ordered before the arrival that publishes them.
FV_DEV void publish(uint32_t bar, int lane) {
    tmem_st_wait();
    tc_fence_before();
    warp_arrive(bar, lane);
}
// P words of the early part (keys [0, kEarlyKeys): 16 kEarlyChunks words from column 0 of the score block) and
// of the late part, out of one 64-word array.
FV_DEV void store_early(uint32_t tS, const uint32_t (&pw)[64]) {
    tmem_st32_at<0>(tS, pw);
    if (kEarlyChunks == 3) tmem_st16_at<32>(tS + 32u, pw);
    if (kEarlyChunks == 4) tmem_st32_at<32>(tS + 32u, pw);
}
FV_DEV void store_late(uint32_t tS, const uint32_t (&pw)[64]) {
    if (kEarlyChunks == 3) tmem_st16_at<48>(tS + 48u, pw);
    else tmem_st32_at<32>(tS + 32u, pw);
}

// What a row carries from key tile to key tile.
struct RowState {
    float m, l;  // reference (base-2 domain, -inf = none yet) and sum of P against it
};

// The careful way through one key tile (or through its late part): masks honoured, exact row maxima
// first, the reference moved where it is missing or more than 2^8 behind, O and the row sum brought
// to the new reference, P evaluated on the MUFU path (an invisible column gives an exact zero).  Kept
// OUT OF LINE on purpose: it runs on the first tile of an item, on tiles a mask cuts through, on a
// segment's last partial tile and when a guard trips, and inlined it more than doubled the code the
// hot loop is spread over (instruction-fetch stalls tripled).
//   late_only: the early part of P is already with the issuer (stored against the old reference);
//   its product must have finished before O is touched -- the caller has waited for pv_early.
//   have_o: O holds products of this item (earlier tiles, or this tile's early part).
static __device__ __noinline__ void careful_tile(uint32_t tS, uint32_t tO, uint32_t bt, Cols cols, float sl2, bool late_only,
                                          bool have_o, int lane, RowState* rs) {
    float m = rs->m, l = rs->l;
    const int first = late_only ? kEarlyChunks : 0;
    float mx = neg_inf();
#pragma unroll 1
    for (int c = first; c < 4; c++) {
        uint32_t u[32];
        load_chunk(tS, c, u);
        land_chunk(u);
        cols.hide(u, 32 * c);
        mx = fmaxf(mx, max32(u));
    }
    const float cand = mx * sl2;
    float a = 1.f;
    if (cand > m + 8.f) {   // (-inf + 8 = -inf: any finite maximum replaces a missing reference)
        a = ex2(m - cand);  // 0 when there was none
        m = cand;
        l *= a;
    }
    if (have_o && __any_sync(kFullWarp, a != 1.f)) {
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
    const float noff = (m == neg_inf()) ? 0.f : -m;  // a row that still sees nothing: P = 2^-inf = 0
    const uint64_t s2 = pack_f32x2(sl2, sl2), nf = pack_f32x2(noff, noff);
    // Chunk by chunk: P of chunk c (16 words at column 16 c) only overwrites scores that have been read.
#pragma unroll 1
    for (int c = first; c < 4; c++) {
        uint32_t u[32], pw[16];
        load_chunk(tS, c, u);
        land_chunk(u);
        cols.hide(u, 32 * c);
        uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
        float top = 0.f;
        exp32<false>(u, pw, s2, nf, acc0, acc1, top);
        l += part_sum<false>(acc0, acc1, top);
        tmem_st16(tS + 16u * (uint32_t)c, pw);
        if (kEarlyChunks < 4 && c == kEarlyChunks - 1) publish(bt + Smem::p_early, lane);
    }
    publish(bt + Smem::p_ready, lane);
    rs->m = m;
    rs->l = l;
}

// 32 columns of one output row: O / l (+ the earlier pass' share), to bf16 or f32.
// A thread holds 32 columns of ITS row; stored as they are, a warp's 16-byte stores would touch 32 rows (32
// lines) each, and the store path takes about a cycle per line and instruction: 8 000 cycles per item for both
// row tiles, which items of a few key tiles (cross-attention) cannot hide.  So the 16-byte pieces are first
// transposed inside groups of G lanes (G = pieces per row: 4 for bf16, 8 for f32): afterwards piece k of a lane
// is piece (lane % G) of the row of lane k of its group, and store number k of a warp writes 32 / G rows' whole
// 64- or 128-byte runs.
template <int G>
FV_DEV void transpose_pieces(uint4 (&p)[G], int lane) {
#pragma unroll
    for (int d = G / 2; d > 0; d >>= 1) {
        const bool hi = (lane & d) != 0;
#pragma unroll
        for (int i = 0; i < G; i++) {
            if (i & d) continue;
            const uint4 send = hi ? p[i] : p[i | d];
            uint4 recv;
            recv.x = __shfl_xor_sync(kFullWarp, send.x, d);
            recv.y = __shfl_xor_sync(kFullWarp, send.y, d);
            recv.z = __shfl_xor_sync(kFullWarp, send.z, d);
            recv.w = __shfl_xor_sync(kFullWarp, send.w, d);
            if (hi) p[i] = recv;
            else p[i | d] = recv;
        }
    }
}

// Where the rows of an item's plane go: element offset of row r is plane_el + r * row_stride (BHSD, or the
// merged-heads [b, s, h * d] layout).
struct OutRows {
    size_t plane_el;
    size_t row_stride;
};
// What the item's output stage needs of the job, by value (it runs out of line).
struct OutJob {
    void* out;
    const float* prev_o;
    const float* prev_lse;
    float* lse_out;
    int sq, out_heads, out_is_bf16;
};

// Columns [32 q, 32 q + 32) of the warp's 32 rows (lane = row qr; rows at or past sq are not stored).  Warp-collective.
FV_DEV void store_cols32(const OutJob& jb, const uint32_t (&o)[32], float inv, float prev_w, const float* prev_row,
                         const OutRows& rows, int q, int qr, int lane) {
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
        uint4 p[4];
#pragma unroll
        for (int c = 0; c < 4; c++)
            p[c] = make_uint4(pack_bf16x2(f[8 * c], f[8 * c + 1]), pack_bf16x2(f[8 * c + 2], f[8 * c + 3]),
                              pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), pack_bf16x2(f[8 * c + 6], f[8 * c + 7]));
        transpose_pieces<4>(p, lane);
        const int l = lane & 3;
        unsigned short* base = reinterpret_cast<unsigned short*>(jb.out) + rows.plane_el + 32 * q + 8 * l;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int r = qr - l + k;
            if (r < jb.sq) *reinterpret_cast<uint4*>(base + (size_t)r * rows.row_stride) = p[k];
        }
    } else {
        uint4 p[8];
#pragma unroll
        for (int c = 0; c < 8; c++)
            p[c] = make_uint4(__float_as_uint(f[4 * c]), __float_as_uint(f[4 * c + 1]), __float_as_uint(f[4 * c + 2]),
                              __float_as_uint(f[4 * c + 3]));
        transpose_pieces<8>(p, lane);
        const int l = lane & 7;
        float* base = reinterpret_cast<float*>(jb.out) + rows.plane_el + 32 * q + 4 * l;
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const int r = qr - l + k;
            if (r < jb.sq) *reinterpret_cast<uint4*>(base + (size_t)r * rows.row_stride) = p[k];
        }
    }
}

// The item's output: O / row sum (merged with an earlier pass' row where there is one), the row's log-sum-exp.
// Out of line like careful_tile: it runs once per item, and inlined its registers (two 32-column buffers, the
// transposed pieces) would be allocated against the hot loop's.  Warp-collective.
// (`jb` by value: read through the kernel's parameter pointer from out here, its fields cost a load each and the
// stage ran 60 % longer; `job`, `tile`, `step`, `stamp` only serve the bring-up stamps.)
static __device__ __noinline__ void write_item(const Job& job, const OutJob jb, uint32_t tO, int plane, int qr, float m,
                                               float l, bool have_o, int lane, int tile, uint32_t step, bool stamp) {
    const bool live = qr < jb.sq;  // rows past sq only take part in the warp-collective TMEM loads
    float inv = l > 0.f ? 1.f / l : 0.f;
    const float lse = (l > 0.f && (jb.lse_out || jb.prev_o)) ? m + log2f(l) : neg_inf();  // (only where it is written or merged)
    const size_t rowi = (size_t)plane * jb.sq + (live ? qr : 0);
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
            if (jb.lse_out) jb.lse_out[rowi] = lse_all;
        } else if (jb.lse_out) {
            jb.lse_out[rowi] = lse;
        }
    }
    OutRows rows{(size_t)plane * jb.sq * kD, (size_t)kD};
    if (jb.out_heads > 0) {
        const int bb = plane / jb.out_heads, hh = plane - bb * jb.out_heads;
        rows.plane_el = ((size_t)bb * jb.sq * jb.out_heads + hh) * kD;
        rows.row_stride = (size_t)jb.out_heads * kD;
    }
    const float* prev_row = (live && jb.prev_o) ? jb.prev_o + rowi * kD : nullptr;  // (the earlier pass is BHSD)
    // Two buffers: the next 32 columns are on their way from TMEM while these are scaled and stored.
    uint32_t oa[32], ob[32];
    if (have_o) {  // warp-uniform
        tmem_ld32_issue(tO, oa);
    } else {
#pragma unroll
        for (int c = 0; c < 32; c++) oa[c] = ob[c] = 0u;
    }
#pragma unroll 1
    for (int h = 0; h < 2; h++) {
        if (have_o) {
            tmem_ld_wait();
            tmem_pin(oa);
            tmem_ld32_issue(tO + 32u * (2 * h + 1), ob);
        }
        store_cols32(jb, oa, inv, prev_w, prev_row ? prev_row + 32 * (2 * h) : nullptr, rows, 2 * h, qr, lane);
        if (h == 0 && stamp && have_o) FV_TR(job, tile, step, 4);
        if (have_o) {
            tmem_ld_wait();
            tmem_pin(ob);
            if (h == 0) tmem_ld32_issue(tO + 64u, oa);
        }
        store_cols32(jb, ob, inv, prev_w, prev_row ? prev_row + 32 * (2 * h + 1) : nullptr, rows, 2 * h + 1, qr, lane);
        if (h == 0 && stamp && have_o) FV_TR(job, tile, step, 5);
    }
    if (stamp && have_o) FV_TR(job, tile, step, 7);
}

template <bool MASKED>
FV_DEV void softmax_warp(const Job& jb, uint32_t sbase, uint32_t tmem, int warp, int lane, const Waiter& wait) {
    const int tile = warp >> 2, quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lanes = tmem + ((uint32_t)(quad * 32) << 16);
    const uint32_t tS = lanes + tmem_scores((uint32_t)tile);  // this row's scores (and P)
    const uint32_t tO = lanes + tmem_output((uint32_t)tile);  // its output accumulator
    const uint32_t bt = sbase + 8u * (uint32_t)tile;  // + Smem::{s_ready, p_early, p_ready, pv_early, o_ready}: this row tile's barriers
    const float sl2 = jb.sl2;
    uint32_t s_count = 0, o_count = 0;

    Deal deal;
    int i = deal.next(jb);
    Item it = item_at(jb, max(i, 0));
    while (i >= 0) {
        const int qr = it.q0 + kRowTile * tile + row;  // this thread's row inside the plane
        const Span cta_span = span_of<MASKED>(jb, global_row(jb, it.q0), global_row(jb, min(it.q0 + kItemRows, jb.sq) - 1));
        const Span row_span = span_of<MASKED>(jb, global_row(jb, qr), global_row(jb, qr));
        RowState rs{neg_inf(), 0.f};
        int seen = 0;
        if (jb.prev_o && qr < jb.sq) {
            // A later pass merges the earlier pass' f32 row in its epilogue.  Each thread reads its own row there
            // (512 bytes, four lines that no other thread shares), one dependent DRAM round trip per 32 columns on
            // the item's critical path: asked for now, the lines are in L2 by then.
            const float* pr = jb.prev_o + ((size_t)it.plane * jb.sq + qr) * kD;
#pragma unroll
            for (int c = 0; c < 4; c++) asm volatile("prefetch.global.L2 [%0];" ::"l"(pr + 32 * c));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(jb.prev_lse + (size_t)it.plane * jb.sq + qr));
        }
        KeyWalk<MASKED> walk;
        KeyTile kt;
        while (walk.next(jb, cta_span, kt)) {
            // (warp-uniform outcomes: the TMEM instructions below are warp-collective)
            if (!__all_sync(kFullWarp, wait(bt + Smem::s_ready, s_count & 1u))) return;
            s_count++;
            tc_fence_after();
            const bool tr = quad == 0 && lane == 0;
            if (tr) FV_TR(jb, tile, s_count - 1u, 0);

            Cols cols{0, kt.valid, 0, kt.valid == kKeyTile};
            if constexpr (MASKED) {
                cols.lo = row_span.lo - kt.k0;
                cols.hi = min(row_span.hi - kt.k0, kt.valid);
                cols.sink = min(row_span.sink - kt.k0, kt.valid);
                cols.whole = (cols.lo <= 0 && cols.hi >= kKeyTile) || cols.sink >= kKeyTile;
            }
            // The hot path takes whole tiles (warp-uniform choice: everything below is warp-collective); tiles a
            // mask or a segment's end cuts go the careful way.  A row without a reference yet (the first tile of
            // an item, or a row that has only met invisible tiles so far: O and its sum are still zero) takes the
            // maximum of its first 32 scores as one -- any reference is exact once O is divided by the row sum,
            // and the guard below catches a row whose later scores outgrow it by 2^40.
            bool hot = __all_sync(kFullWarp, cols.whole);
            if (hot) {
                // Four 32-column chunks, the next one on its way from TMEM while this one's exponentials run.
                uint32_t u0[32], u1[32], pw[64];
                load_chunk(tS, 0, u0);
                land_chunk(u0);
                if (rs.m == neg_inf()) rs.m = max32(u0) * sl2;
                const uint64_t s2 = pack_f32x2(sl2, sl2), nf = pack_f32x2(-rs.m, -rs.m);
                uint64_t acc0 = pack_f32x2(0.f, 0.f), acc1 = acc0;
                float top = 0.f;
                if (tr) FV_TR(jb, tile, s_count - 1u, 1);
                load_chunk(tS, 1, u1);
                exp32<true>(u0, pw, s2, nf, acc0, acc1, top);
                land_chunk(u1);
                load_chunk(tS, 2, u0);
                exp32<true>(u1, pw + 16, s2, nf, acc0, acc1, top);
                land_chunk(u0);
                load_chunk(tS, 3, u1);
                if (kEarlyChunks >= 3) exp32<true>(u0, pw + 32, s2, nf, acc0, acc1, top);
                if (kEarlyChunks == 4) {
                    land_chunk(u1);
                    exp32<true>(u1, pw + 48, s2, nf, acc0, acc1, top);
                }
                const float sum0 = part_sum<true>(acc0, acc1, top);
                if (tr) FV_TR(jb, tile, s_count - 1u, 2);
                if (__any_sync(kFullWarp, !(sum0 <= kGuard))) {
                    if (kEarlyChunks < 4) land_chunk(u1);  // (nothing may be in flight into registers when the call is made)
                    hot = false;              // nothing of this tile is stored: the careful way, whole tile
                } else if (kEarlyChunks == 4) {
                    store_early(tS, pw);      // the whole of P in one hand-over
                    publish(bt + Smem::p_ready, lane);
                    if (tr) FV_TR(jb, tile, s_count - 1u, 6);
                    rs.l += sum0;
                } else {
                    store_early(tS, pw);
                    publish(bt + Smem::p_early, lane);
                    if (tr) FV_TR(jb, tile, s_count - 1u, 3);
                    acc0 = acc1 = pack_f32x2(0.f, 0.f);
                    top = 0.f;
                    if (kEarlyChunks == 2) exp32<true>(u0, pw + 32, s2, nf, acc0, acc1, top);
                    land_chunk(u1);
                    if (tr) FV_TR(jb, tile, s_count - 1u, 4);
                    exp32<true>(u1, pw + 48, s2, nf, acc0, acc1, top);
                    const float sum1 = part_sum<true>(acc0, acc1, top);
                    if (tr) FV_TR(jb, tile, s_count - 1u, 5);
                    if (__any_sync(kFullWarp, !(sum1 <= kGuard))) {
                        // The early part went out against the old reference and its product may be running:
                        // wait for it (the issuer signals every early product), then the careful way for the
                        // late part, whose scores (columns kEarlyKeys-127 of S) are untouched.
                        rs.l += sum0;
                        if (!__all_sync(kFullWarp, wait(bt + Smem::pv_early, (s_count - 1u) & 1u))) return;
                        tc_fence_after();
                        careful_tile(tS, tO, bt, cols, sl2, true, true, lane, &rs);
                    } else {
                        store_late(tS, pw);
                        publish(bt + Smem::p_ready, lane);
                        if (tr) FV_TR(jb, tile, s_count - 1u, 6);
                        rs.l += sum0 + sum1;
                    }
                }
            }
            if (!hot) careful_tile(tS, tO, bt, cols, sl2, false, seen > 0, lane, &rs);
            seen++;
        }

        // ------------------------------------------------------------------------- the item's output
        // (the next item is looked up now, while the last product runs, not after the output is written)
        const int plane = it.plane;
        i = deal.next(jb);
        if (i >= 0) it = item_at(jb, i);
        if (seen > 0) {
            if (!__all_sync(kFullWarp, wait(bt + Smem::o_ready, o_count & 1u))) return;
            o_count++;
            tc_fence_after();
            if (quad == 0 && lane == 0) FV_TR(jb, tile, s_count - 1u, 3);
        }
        write_item(jb, OutJob{jb.out, jb.prev_o, jb.prev_lse, jb.lse_out, jb.sq, jb.out_heads, jb.out_is_bf16}, tO, plane, qr,
                   rs.m, rs.l, seen > 0, lane, tile, s_count - 1u, quad == 0 && lane == 0);
        // The next item's first P.V overwrites O.  The issuer issues it only after all four warps of the
        // row tile have arrived at p_ready for that item's first key tile, and a warp gets there only
        // after its loads above have completed.
    }
}

// --------------------------------------------------------------------------------------- loader
template <bool MASKED>
FV_DEV void loader_thread(const CUtensorMap* mq, const CUtensorMap* mk, const CUtensorMap* mv, const Job& jb,
                          uint32_t sbase, const Waiter& wait) {
    uint32_t qn = 0, kvn = 0;  // Q tiles and K/V pairs loaded so far
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
    // Pair number p of the run lives in pair slot p % kKvPairs: first tile V of the previous key tile (absent in
    // an item's first pair), second tile K of this key tile (absent in its last pair).  One barrier per pair.
    auto load_pair = [&](const KeyTile* vt, const KeyTile* kt, int plane) -> bool {
        const uint32_t slot = kvn % kKvPairs, use = kvn / kKvPairs;
        if (use > 0 && !wait(sbase + Smem::kv_free + 8u * slot, (use - 1u) & 1u)) return false;
        const uint32_t dst = sbase + Smem::kv + slot * 2u * kSlotBytes, bar = sbase + Smem::kv_full + 8u * slot;
        mbar_expect_tx(bar, (vt ? kSlotBytes : 0u) + (kt ? kSlotBytes : 0u));
        if (vt) {
            tma_load4(dst, mv, bar, 0, vt->t * kKeyTile, plane, vt->seg);
            tma_load4(dst + kPanelBytes, mv, bar, 64, vt->t * kKeyTile, plane, vt->seg);
        }
        if (kt) {
            tma_load4(dst + kSlotBytes, mk, bar, 0, kt->t * kKeyTile, plane, kt->seg);
            tma_load4(dst + kSlotBytes + kPanelBytes, mk, bar, 64, kt->t * kKeyTile, plane, kt->seg);
        }
        kvn++;
        return true;
    };

    Deal deal;
    int i = deal.next(jb);
    bool ok = true;
    if (i >= 0) ok = load_q(i, 0) && load_q(i, 1);
    for (; ok && i >= 0; i = deal.next(jb)) {
        const int nxt = deal.peek(jb);
        // Row tile A of the next item goes into the slot the previous item's tile B left long ago.
        if (nxt >= 0) ok = load_q(nxt, 0);
        const Item it = item_at(jb, i);
        const Span sp = span_of<MASKED>(jb, global_row(jb, it.q0), global_row(jb, min(it.q0 + kItemRows, jb.sq) - 1));
        KeyWalk<MASKED> walk;
        KeyTile kt;
        KeyTile prev;
        bool have_prev = false;
        while (ok && walk.next(jb, sp, kt)) {
            ok = load_pair(have_prev ? &prev : nullptr, &kt, it.plane);
            prev = kt;
            have_prev = true;
        }
        if (ok && have_prev) ok = load_pair(&prev, nullptr, it.plane);
        // Tile B of the next item takes the slot of this item's tile A, free after its last Q.K^T.
        if (ok && nxt >= 0) ok = load_q(nxt, 1);
    }
    // Copies in flight must land before the CTA's shared memory goes away.  After a clean run the
    // issuer has waited on every one of these phases already and the loops fall straight through.
    for (uint32_t s = 0; s < (uint32_t)kQSlots && s < qn; s++) {
        const uint32_t last = ((qn - 1u - s) / kQSlots) * kQSlots + s;  // last load that used slot s
        mbar_drain(sbase + Smem::q_full + 8u * s, (last / kQSlots) & 1u);
    }
    for (uint32_t s = 0; s < (uint32_t)kKvPairs && s < kvn; s++) {
        const uint32_t last = ((kvn - 1u - s) / kKvPairs) * kKvPairs + s;
        mbar_drain(sbase + Smem::kv_full + 8u * s, (last / kKvPairs) & 1u);
    }
}

// --------------------------------------------------------------------------------------- issuer
// Ring positions are plain counters: load number c lives in slot c % slots, and it is the
// (c / slots)-th use of that slot, whose barrier phase has the parity of that quotient.
FV_DEV uint32_t kv_slot_addr(uint32_t sbase, uint32_t c) { return sbase + Smem::kv + (c % kKvSlots) * kSlotBytes; }

// P_t(j) . V(j) into O_t in two steps, keys 0-63 as soon as that half of P is stored, then the rest.
// `pc` counts the P tiles of this row tile consumed so far (its parity is the phase of p_early,
// p_ready and pv_early).  The first product of an item overwrites O; the softmax threads of the
// previous item have finished reading it by the time they have stored any of the new item's P.
// (An issuer that serves the two row tiles out of order, probing their barriers without blocking, was
// tried: its probes compete with the MMAs' operand reads for shared memory and it ran 23 % slower.)
FV_DEV bool issue_output(const Job& jb, uint32_t sbase, uint32_t t, uint32_t tmem, uint64_t vd, bool fresh, uint32_t pc,
                         const Waiter& wait) {
    const uint32_t bt = sbase + 8u * t, tO = tmem + tmem_output(t), tP = tmem + tmem_scores(t);
    if (kEarlyKeys < 128) {
        if (!wait(bt + Smem::p_early, pc & 1u)) return false;
        FV_TR(jb, 2, pc, 1 + 3 * t);
        tc_fence_after();
        output_mma_early(tO, tP, vd, fresh);
        umma_commit(bt + Smem::pv_early);
    }
    if (!wait(bt + Smem::p_ready, pc & 1u)) return false;
    FV_TR(jb, 2, pc, 2 + 3 * t);
    tc_fence_after();
    if (kEarlyKeys == 128) output_mma_early(tO, tP, vd, fresh);
    else output_mma_late(tO, tP, vd);
    return true;
}

// The issuer: one thread, strictly in order.  Step j of an item (j = 0 .. n) is, for row tile t = A then B:
// O_t += P_t(j-1) . V(j-1) for j > 0, then S_t = Q_t . K(j)^T for j < n.  The K/V ring is used in pairs
// [V(j-1) | K(j)]: ONE wait for the pair's arrival and ONE commit that frees it per step, because every wait and
// every commit is a point where this thread can stall while the tensor pipe's short queue runs dry.
// (Two issuer threads, one per row tile, were tried: the two tiles' softmaxes then run in phase, share the MUFU
// pipe for their whole length and the products wait for both -- 20 % slower.  The single in-order thread is what
// keeps the tiles half a period apart.)
template <bool MASKED>
FV_DEV void issuer_thread(const Job& jb, uint32_t sbase, uint32_t tmem, const Waiter& wait) {
    uint32_t qn = 0;   // Q tiles consumed (two per item)
    uint32_t pn = 0;   // K/V pairs consumed
    uint32_t pc = 0;   // P tiles consumed per row tile
    Deal deal;
    for (int i = deal.next(jb); i >= 0; i = deal.next(jb)) {
        const Item it = item_at(jb, i);
        const Span sp = span_of<MASKED>(jb, global_row(jb, it.q0), global_row(jb, min(it.q0 + kItemRows, jb.sq) - 1));
        const int n = count_tiles<MASKED>(jb, sp);
        const uint32_t qa = qn % kQSlots, qb = (qn + 1u) % kQSlots;  // this item's Q slots
        const uint32_t qa_par = (qn / kQSlots) & 1u, qb_par = ((qn + 1u) / kQSlots) & 1u;
        qn += 2;
        if (n == 0) {
            // No key of any segment is visible to these rows.  The Q tiles were loaded all the same: let
            // them land before their slots are handed back.
            if (!wait(sbase + Smem::q_full + 8u * qa, qa_par) || !wait(sbase + Smem::q_full + 8u * qb, qb_par)) break;
            mbar_arrive(sbase + Smem::q_free + 8u * qa);
            mbar_arrive(sbase + Smem::q_free + 8u * qb);
            continue;
        }
        const uint64_t qd_a = umma_desc_sw128(sbase + Smem::q + qa * kSlotBytes, 16, 1024);
        const uint64_t qd_b = umma_desc_sw128(sbase + Smem::q + qb * kSlotBytes, 16, 1024);
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j <= n; j++) {
            const uint32_t slot = pn % kKvPairs;
            const uint32_t pair = sbase + Smem::kv + slot * 2u * kSlotBytes;  // V(j-1) in its first tile, K(j) in its second
            if (!wait(sbase + Smem::kv_full + 8u * slot, (pn / kKvPairs) & 1u)) { ok = false; break; }
            tc_fence_after();
            const uint64_t vd = umma_desc_sw128(pair, kPanelBytes, 1024);
            const uint64_t kd = umma_desc_sw128(pair + kSlotBytes, 16, 1024);
            if (j > 0) FV_TR(jb, 2, pc, 0);
#pragma unroll
            for (uint32_t t = 0; t < 2; t++) {
                if (j > 0 && !issue_output(jb, sbase, t, tmem, vd, j == 1, pc, wait)) { ok = false; break; }
                if (j == n) {
                    umma_commit(sbase + Smem::o_ready + 8u * t);
                    continue;
                }
                if (j == 0) {  // (tile B of an item is loaded late, see loader_thread: it is waited for where it is first used)
                    if (!wait(sbase + Smem::q_full + 8u * (t ? qb : qa), t ? qb_par : qa_par)) { ok = false; break; }
                    tc_fence_after();
                }
                scores_mma(tmem + tmem_scores(t), t ? qd_b : qd_a, kd);
                umma_commit(sbase + Smem::s_ready + 8u * t);
                if (j > 0) FV_TR(jb, 2, pc, 3 + 3 * t);
                if (j == n - 1) umma_commit(sbase + Smem::q_free + 8u * (t ? qb : qa));
            }
            if (!ok) break;
            umma_commit(sbase + Smem::kv_free + 8u * slot);
            pn++;
            if (j > 0) pc++;
        }
        if (!ok) break;
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
            mbar_init(sbase + Smem::p_early + 8u * t, 4);  // the row tile's four softmax warps
            mbar_init(sbase + Smem::p_ready + 8u * t, 4);
            mbar_init(sbase + Smem::pv_early + 8u * t, 1);
            mbar_init(sbase + Smem::o_ready + 8u * t, 1);
        }
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
        asm volatile("setmaxnreg.inc.sync.aligned.u32 216;" ::: "memory");
        softmax_warp<MASKED>(jb, sbase, tmem, warp, lane, Waiter{jb, sbase, 3});
    } else {
        // (one setmaxnreg for the whole warpgroup: warps 8-11 execute this very instruction together)
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;" ::: "memory");
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

// Video Sparse Attention (VSA) for Wan on sm_100a: tile + mean-pool, coarse tile attention with
// the reference's exact selection arithmetic, top-k tile selection, fine sparse attention over the
// selected 64-key tiles on tcgen05 / TMEM, and the gated combine fused into its epilogue.
//
// Stands in for rt::vsa::vsa_attention_device (crates/fastvideo-cudarc/src/rt/vsa.rs:358-470) and the
// launchers it calls (crates/fastvideo-cudarc/src/rt/ops.rs:811-923,1074-1383,1554-1619;
// crates/fastvideo-cudarc/src/rt/attn_dc.rs:275-604), with the host twin rt/vsa.rs:116-262 as the
// arithmetic to match:
//   tile means   in-order f32 sum over a tile's real slots, then one f32 division by the real count
//   scores       f64 dot of the f32 means (products exact, summed in index order) * f64(scale) -> f32
//   selection    the top-k scores per query tile, ties to the lower tile index; emitted ASCENDING by
//                tile index (the reference's host emits by score; same set)
//   coarse       softmax over tiles in f64, out accumulated in f32 in tile order
//   fine         softmax(q k^T * scale) v over the selected tiles' real keys, bf16 MMA, f32 softmax
//   combine      out[token] = coarse[tile] * gate[token] + fine   (f32, separate multiply and add)
#include "fv_ptx.cuh"
#include "fv_runtime.h"
#include <cuda.h>
#include <cuda_bf16.h>
#include <math.h>
#include <string.h>
#include <algorithm>
#include <vector>

namespace fvvsa {

constexpr int TE = 64;  // slots per tile (4 x 4 x 4)
constexpr int kD = 128;

struct Plan {
    int gt, gh, gw, nt, seq, padded;
    std::vector<int32_t> slot_src;
    std::vector<uint32_t> token_slot, block_sizes;
    int device;
    int32_t* d_slot_src;
    uint32_t* d_block_sizes;
};

// ------------------------------------------------------------------ 1. tile + pool
// grid (nt, bh), 192 threads: group g = tid / 64 handles q, k or v; thread owns 2 consecutive dims and
// walks the tile's 64 slots in order (the in-order f32 sum the selection arithmetic needs).
__global__ void __launch_bounds__(192) vsa_prep_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                       const __nv_bfloat16* __restrict__ v, const int32_t* __restrict__ slot_src,
                                                       const uint32_t* __restrict__ block_sizes, int seq, int nt,
                                                       __nv_bfloat16* __restrict__ qt, __nv_bfloat16* __restrict__ kt,
                                                       __nv_bfloat16* __restrict__ vt, float* __restrict__ means) {
    const int tile = blockIdx.x, bh = blockIdx.y, g = threadIdx.x >> 6, t = threadIdx.x & 63;
    const __nv_bfloat16* src = (g == 0 ? q : g == 1 ? k : v) + (size_t)bh * seq * kD;
    __nv_bfloat16* dst = (g == 0 ? qt : g == 1 ? kt : vt) + ((size_t)bh * nt + tile) * TE * kD;
    const int n = (int)block_sizes[tile];
    float s0 = 0.f, s1 = 0.f;
#pragma unroll 8
    for (int slot = 0; slot < TE; slot++) {
        uint32_t w = 0u;
        if (slot < n) {
            const int token = slot_src[tile * TE + slot];
            w = *reinterpret_cast<const uint32_t*>(src + (size_t)token * kD + 2 * t);
            s0 = __fadd_rn(s0, __uint_as_float(w << 16));
            s1 = __fadd_rn(s1, __uint_as_float(w & 0xffff0000u));
        }
        *reinterpret_cast<uint32_t*>(dst + (size_t)slot * kD + 2 * t) = w;
    }
    float2 m = make_float2(0.f, 0.f);
    if (n > 0) m = make_float2(__fdiv_rn(s0, (float)n), __fdiv_rn(s1, (float)n));
    // means: [3][bh, nt, 128]
    float* mp = means + ((size_t)g * gridDim.y * nt + (size_t)bh * nt + tile) * kD + 2 * t;
    *reinterpret_cast<float2*>(mp) = m;
}

// ------------------------------------------------------------------ 2. coarse scores (f64, in order)
// grid (ceil(nt/64), ceil(nt/64), bh), 256 threads: a 64 x 64 block of (query tile, key tile) pairs per CTA, a 4 x 4
// patch per thread (shared-memory reads, not the FMAs, bound the 1 x 1 version).  Dynamic smem: 2 x 64 x 129 doubles.
constexpr int kScoreTile = 64;
constexpr size_t kScoreSmem = 2 * (size_t)kScoreTile * (kD + 1) * sizeof(double);
__global__ void __launch_bounds__(256) vsa_scores_kernel(const float* __restrict__ qc, const float* __restrict__ kc, int nt,
                                                         float scale, float* __restrict__ scores) {
    // the means widened to f64 once, on the way into shared memory (a conversion per use would cost more than the FMA)
    extern __shared__ double score_smem[];
    double (*qs)[kD + 1] = reinterpret_cast<double (*)[kD + 1]>(score_smem);
    double (*ks)[kD + 1] = reinterpret_cast<double (*)[kD + 1]>(score_smem + (size_t)kScoreTile * (kD + 1));
    const int bh = blockIdx.z, q0 = blockIdx.y * kScoreTile, k0 = blockIdx.x * kScoreTile;
    for (int e = threadIdx.x; e < kScoreTile * kD; e += 256) {
        const int r = e / kD, c = e % kD;
        qs[r][c] = (q0 + r < nt) ? (double)qc[((size_t)bh * nt + q0 + r) * kD + c] : 0.0;
        ks[r][c] = (k0 + r < nt) ? (double)kc[((size_t)bh * nt + k0 + r) * kD + c] : 0.0;
    }
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    double acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.0;
#pragma unroll 4
    for (int d = 0; d < kD; d++) {
        double qv[4], kv[4];
#pragma unroll
        for (int a = 0; a < 4; a++) {
            qv[a] = qs[ty + 16 * a][d];
            kv[a] = ks[tx + 16 * a][d];
        }
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int b = 0; b < 4; b++) acc[a][b] = fma(qv[a], kv[b], acc[a][b]);  // product exact: == multiply then add, in index order
    }
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int qi = q0 + ty + 16 * a, kj = k0 + tx + 16 * b;
            if (qi < nt && kj < nt) scores[((size_t)bh * nt + qi) * nt + kj] = (float)(acc[a][b] * (double)scale);
        }
}

// ------------------------------------------------------------------ 3. coarse attention over tiles
// grid (ceil(nt / kCoarseQT), bh), 128 threads (thread = output dim).  One CTA serves kCoarseQT query tiles so that each
// row of the pooled V is read from L2 once per kCoarseQT outputs.  Softmax weights in f64 (max, exp, sum, divide as the
// host does), kept as f32; out accumulated in f32 in tile order.  Dynamic smem: kCoarseQT * nt floats + nt doubles.
constexpr int kCoarseQT = 4;
__global__ void __launch_bounds__(128) vsa_coarse_kernel(const float* __restrict__ scores, const float* __restrict__ vc, int nt,
                                                         float* __restrict__ coarse) {
    extern __shared__ double coarse_smem[];
    double* ebuf = coarse_smem;                               // [nt]
    float* wts = reinterpret_cast<float*>(coarse_smem + nt);  // [kCoarseQT][nt]
    __shared__ float redf[4];
    __shared__ double redd[4];
    const int qt0 = blockIdx.x * kCoarseQT, bh = blockIdx.y, t = threadIdx.x, lane = t & 31, warp = t >> 5;
#pragma unroll 1
    for (int q = 0; q < kCoarseQT; q++) {
        const int qt = qt0 + q;
        if (qt >= nt) break;  // CTA-uniform
        const float* s = scores + ((size_t)bh * nt + qt) * nt;
        float m = -INFINITY;
        for (int i = t; i < nt; i += 128) m = fmaxf(m, s[i]);
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        __syncthreads();  // redf / redd / ebuf of the previous query tile are no longer read
        if (lane == 0) redf[warp] = m;
        __syncthreads();
        m = fmaxf(fmaxf(redf[0], redf[1]), fmaxf(redf[2], redf[3]));
        double z = 0.0;
        for (int i = t; i < nt; i += 128) {
            const double e = exp((double)(s[i] - m));
            ebuf[i] = e;
            z += e;
        }
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(0xffffffffu, z, o);
        if (lane == 0) redd[warp] = z;
        __syncthreads();
        z = (redd[0] + redd[1]) + (redd[2] + redd[3]);
        for (int i = t; i < nt; i += 128) wts[(size_t)q * nt + i] = (float)(ebuf[i] / z);
    }
    __syncthreads();
    float acc[kCoarseQT];
#pragma unroll
    for (int q = 0; q < kCoarseQT; q++) acc[q] = 0.f;
    const float* vch = vc + (size_t)bh * nt * kD + t;
    const int nq = min(kCoarseQT, nt - qt0);
#pragma unroll 4
    for (int kt = 0; kt < nt; kt++) {
        const float v = vch[(size_t)kt * kD];
#pragma unroll
        for (int q = 0; q < kCoarseQT; q++)
            if (q < nq) acc[q] = __fadd_rn(acc[q], __fmul_rn(wts[(size_t)q * nt + kt], v));
    }
#pragma unroll
    for (int q = 0; q < kCoarseQT; q++)
        if (q < nq) coarse[((size_t)bh * nt + qt0 + q) * kD + t] = acc[q];
}

// ------------------------------------------------------------------ 4. top-k tiles per query tile
// grid (nt, bh), 256 threads; dynamic smem: nt keys.  Exact selection: the k largest scores, ties to
// the lower index, written in ascending index order.
__device__ __forceinline__ uint32_t order_key(float f) {  // ascending unsigned order == f32 total order
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ int block_sum(int v, int* red) {  // 256 threads; all get the total
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    int tot = 0;
    for (int w = 0; w < 8; w++) tot += red[w];
    return tot;
}
// exclusive prefix of a 0/1 flag over the block, and the block total
__device__ __forceinline__ int block_excl_scan(bool flag, int* red, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t b = __ballot_sync(0xffffffffu, flag);
    const int within = __popc(b & ((1u << lane) - 1u));
    __syncthreads();
    if (lane == 0) red[warp] = __popc(b);
    __syncthreads();
    int base = 0, tot = 0;
    for (int w = 0; w < 8; w++) {
        if (w < warp) base += red[w];
        tot += red[w];
    }
    *total = tot;
    return base + within;
}
__global__ void __launch_bounds__(256) vsa_topk_kernel(const float* __restrict__ scores, int nt, int topk,
                                                       uint32_t* __restrict__ selected) {
    extern __shared__ uint32_t keys[];
    __shared__ int red[8];
    const int row = blockIdx.x, bh = blockIdx.y, t = threadIdx.x;
    const float* s = scores + ((size_t)bh * nt + row) * nt;
    for (int i = t; i < nt; i += 256) keys[i] = order_key(s[i]);
    __syncthreads();
    // T = the k-th largest key: the largest T with count(key >= T) >= k, built bit by bit
    uint32_t T = 0u;
    for (int b = 31; b >= 0; b--) {
        const uint32_t cand = T | (1u << b);
        int c = 0;
        for (int i = t; i < nt; i += 256) c += keys[i] >= cand;
        if (block_sum(c, red) >= topk) T = cand;
    }
    int c = 0;
    for (int i = t; i < nt; i += 256) c += keys[i] > T;
    const int need_eq = topk - block_sum(c, red);  // how many of the keys equal to T are kept (lowest indices)
    uint32_t* out = selected + ((size_t)bh * nt + row) * topk;
    int eq_seen = 0, written = 0;
    for (int base = 0; base < nt; base += 256) {
        const int i = base + t;
        const uint32_t key = i < nt ? keys[i] : 0u;
        const bool eq = i < nt && key == T;
        int eq_tot, sel_tot;
        const int eq_rank = eq_seen + block_excl_scan(eq, red, &eq_tot);
        const bool sel = i < nt && (key > T || (eq && eq_rank < need_eq));
        const int pos = written + block_excl_scan(sel, red, &sel_tot);
        if (sel && pos < topk) out[pos] = (uint32_t)i;
        eq_seen += eq_tot;
        written += sel_tot;
    }
}

// The same selection with one WARP per row (rows of up to kTopkWarpMax scores): no block-wide barriers.  grid
// (ceil(rows / 8), 1), 256 threads; dynamic smem: 8 * nt keys.
constexpr int kTopkWarpMax = 1024;
__global__ void __launch_bounds__(256) vsa_topk_warp_kernel(const float* __restrict__ scores, int rows, int nt, int topk,
                                                            uint32_t* __restrict__ selected) {
    extern __shared__ uint32_t wkeys[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 8 + warp;
    if (row >= rows) return;  // warp-uniform; no block barrier below
    uint32_t* keys = wkeys + (size_t)warp * nt;
    const float* s = scores + (size_t)row * nt;
    for (int i = lane; i < nt; i += 32) keys[i] = order_key(s[i]);
    __syncwarp();
    uint32_t T = 0u;
    for (int b = 31; b >= 0; b--) {
        const uint32_t cand = T | (1u << b);
        int c = 0;
        for (int i = lane; i < nt; i += 32) c += keys[i] >= cand;
        if (__reduce_add_sync(0xffffffffu, c) >= topk) T = cand;
    }
    int c = 0;
    for (int i = lane; i < nt; i += 32) c += keys[i] > T;
    const int need_eq = topk - __reduce_add_sync(0xffffffffu, c);
    uint32_t* out = selected + (size_t)row * topk;
    int eq_seen = 0, written = 0;
    const uint32_t below = (1u << lane) - 1u;
    for (int base = 0; base < nt; base += 32) {
        const int i = base + lane;
        const uint32_t key = i < nt ? keys[i] : 0u;
        const bool eq = i < nt && key == T;
        const uint32_t eqm = __ballot_sync(0xffffffffu, eq);
        const bool sel = i < nt && (key > T || (eq && eq_seen + __popc(eqm & below) < need_eq));
        const uint32_t selm = __ballot_sync(0xffffffffu, sel);
        const int pos = written + __popc(selm & below);
        if (sel && pos < topk) out[pos] = (uint32_t)i;
        eq_seen += __popc(eqm);
        written += __popc(selm);
    }
}

// ------------------------------------------------------------------ 5. fine attention + combine
// CTA = two query tiles (128 rows) of one head, 6 warps: 0-3 softmax (thread = TMEM lane = row;
// rows 0-63 are tile 2p, rows 64-127 tile 2p+1), 4 list builder + TMA producer, 5 MMA issuer.
// The CTA walks the ascending union of the two tiles' selections, one 64-key tile per step; an
// entry word says which of the two query tiles selected it (the other one's rows get P = 0) and how
// many of its 64 slots are real keys.  TMEM (256 columns, two CTAs per SM): two S buffers at 0 and 64 (64
// columns each; the bf16 P of a step overwrites columns 0-31 of its buffer), O at 128 (128 columns).  Q.K^T runs two
// steps ahead of P.V, so the softmax of step j+1 starts as soon as that of step j ends.
constexpr int kFineThreads = 192;
constexpr int kFineNS = 4;
constexpr uint32_t kKvTileB = 16384;   // 64 x 128 bf16: two 8 KB panels
constexpr uint32_t kKvPanelB = 8192;
constexpr uint32_t kQTileB = 32768;    // 128 x 128 bf16: two 16 KB panels
constexpr uint32_t kQPanelB = 16384;

struct FineParams {
    const uint32_t* selected;     // [bh, nt, topk] ascending
    const uint32_t* block_sizes;  // [nt]
    const int32_t* slot_src;      // [nt*64]
    const float* coarse;          // [bh, nt, 128]
    const __nv_bfloat16* gate;    // [bh, seq, 128] or null (gate of one)
    void* out;                    // [bh, seq, 128]
    int* status;
    int out_is_bf16;
    int bh, nt, topk, seq;
    float sl2;
    int list_cap;
};

__global__ void __launch_bounds__(kFineThreads, 2)
fv_vsa_fine_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ FineParams p) {
#if defined(__CUDA_ARCH_FEAT_SM100_ALL) || defined(__CUDA_ARCH_FEAT_SM103_ALL)
    using namespace fvp;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    const uint32_t sQ = base;
    const uint32_t ring = base + kQTileB;
    const uint32_t bars = ring + kFineNS * kKvTileB;
    const uint32_t b_q = bars;
    const uint32_t b_full = b_q + 8;
    const uint32_t b_empty = b_full + 8 * kFineNS;
    const uint32_t b_s = b_empty + 8 * kFineNS;  // [2]: S buffer ready
    const uint32_t b_p = b_s + 16;               // [2]: P stored in that buffer
    const uint32_t b_od = b_p + 16;              // one phase per P.V
    const uint32_t b_o = b_od + 8;               // the last P.V
    const uint32_t b_drain = b_o + 8;
    const uint32_t tslot = b_drain + 8;
    const uint32_t aflag = tslot + 4;
    const uint32_t nent_a = aflag + 4;
    const uint32_t list_a = bars + 256;
    volatile uint32_t* tslot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tslot - raw));
    volatile int* abort_ptr = reinterpret_cast<volatile int*>(smem_raw + (aflag - raw));
    volatile int* nent_ptr = reinterpret_cast<volatile int*>(smem_raw + (nent_a - raw));
    volatile uint32_t* list = reinterpret_cast<volatile uint32_t*>(smem_raw + (list_a - raw));

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int npair = (p.nt + 1) / 2;
    const int pair = (int)(blockIdx.x % (unsigned)npair), bh = (int)(blockIdx.x / (unsigned)npair);
    const int qt0 = 2 * pair, qt1 = 2 * pair + 1;
    const float NEG = __int_as_float(0xff800000);

    if (tid == 0) {
        mbar_init(b_q, 1);
        for (int i = 0; i < kFineNS; i++) {
            mbar_init(b_full + 8 * i, 1);
            mbar_init(b_empty + 8 * i, 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(b_s + 8 * i, 1);
            mbar_init(b_p + 8 * i, 128);
        }
        mbar_init(b_od, 1);
        mbar_init(b_o, 1);
        mbar_init(b_drain, 1);
        *abort_ptr = (*(volatile int*)p.status != FV_ST_OK) ? 1 : 0;
        mbar_init_fence();
    }
    __syncthreads();
    if (*abort_ptr) return;  // CTA-uniform
    if (warp == 5) tmem_alloc(tslot, 256);
    if (warp == 4) {
        if (lane == 0) {
            tma_prefetch_desc(&tq);
            mbar_expect_tx(b_q, kQTileB);
            tma_load4(sQ, &tq, b_q, 0, qt0 * TE, bh, 0);
            tma_load4(sQ + kQPanelB, &tq, b_q, 64, qt0 * TE, bh, 0);
        }
        // ---- the ascending union of the two selections, with visibility bits (27: tile qt0, 28: tile qt1)
        const uint32_t* la = p.selected + ((size_t)bh * p.nt + qt0) * p.topk;
        const uint32_t* lb = p.selected + ((size_t)bh * p.nt + qt1) * p.topk;
        const int na = p.topk, nb = qt1 < p.nt ? p.topk : 0;
        // both selections are staged in shared memory behind the union area, then merged by one lane
        volatile uint32_t* sa = list + p.list_cap;
        volatile uint32_t* sb = sa + p.topk;
        for (int i = lane; i < na; i += 32) sa[i] = la[i];
        for (int i = lane; i < nb; i += 32) sb[i] = lb[i];
        __syncwarp();
        if (lane == 0) {
            int i = 0, j = 0, n = 0;
            while ((i < na || j < nb) && n < p.list_cap) {
                const uint32_t a = i < na ? sa[i] : 0xffffffffu, b = j < nb ? sb[j] : 0xffffffffu;
                uint32_t e;
                if (a < b) { e = a | (1u << 27); i++; }
                else if (b < a) { e = b | (2u << 27); j++; }
                else { e = a | (3u << 27); i++; j++; }
                list[n++] = e;
            }
            *nent_ptr = n;
        }
        __syncwarp();
        const int n = *nent_ptr;
        for (int i = lane; i < n; i += 32) {
            const uint32_t e = list[i];
            list[i] = e | (min(p.block_sizes[e & 0xFFFFFu], 64u) << 20);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tbase = *tslot_ptr;
    const int nent = *nent_ptr;

    if (warp < 4) {
        // ------------------------------------------------------------ softmax
        WaitCtl ctl{abort_ptr, p.status, 13};
        const int row = warp * 32 + lane, half = row >> 6;
        const uint32_t tl = tbase + ((uint32_t)(warp * 32) << 16);
        const uint32_t tO = tl + 128u;
        const float sl2 = p.sl2;
        float m = NEG, l = 0.f;
        bool ok = true;
#pragma unroll 1
        for (int j = 0; j < nent && ok; j++) {
            const uint32_t e = list[j];
            const int valid = (int)((e >> 20) & 127u);
            const bool vis = ((e >> (27 + half)) & 1u) != 0u;  // warp-uniform: a warp lies inside one half
            const int bsel = j & 1;
            const uint32_t tS = tl + 64u * bsel, tP = tS;
            if (!__all_sync(0xffffffffu, mbar_wait(b_s + 8 * bsel, (j >> 1) & 1, ctl))) { ok = false; break; }
            tc_fence_after();
            uint32_t pw[32];
            if (vis) {
                uint32_t u[64];
                {
                    uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&u[0]);
                    uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&u[32]);
                    tmem_ld32_issue(tS, lo);
                    tmem_ld32_issue(tS + 32u, hi);
                    tmem_ld_wait();
                    tmem_pin(u);
                }
                if (valid < TE) {
#pragma unroll
                    for (int c = 0; c < 64; c++) u[c] = c < valid ? u[c] : __float_as_uint(NEG);
                }
                float x0 = __uint_as_float(u[0]), x1 = __uint_as_float(u[1]);
#pragma unroll
                for (int c = 2; c < 64; c += 2) {
                    x0 = fmaxf(x0, __uint_as_float(u[c]));
                    x1 = fmaxf(x1, __uint_as_float(u[c + 1]));
                }
                const float tm2 = fmaxf(x0, x1) * sl2;
                const bool grow = tm2 > m + 8.0f;
                float a = 1.f;
                if (grow) {
                    a = ex2(m - tm2);
                    m = tm2;
                }
                const float off = (m == NEG) ? 0.f : m;
                // S_j done only implies PV_{j-2} done (Q.K^T runs two steps ahead): wait for PV_{j-1} before touching O
                if (j > 0 && __any_sync(0xffffffffu, grow)) {
                    if (!__all_sync(0xffffffffu, mbar_wait(b_od, (j - 1) & 1, ctl))) { ok = false; break; }
                    tc_fence_after();
#pragma unroll 1
                    for (int q = 0; q < 4; q++) {
                        uint32_t o[32];
                        tmem_ld32_issue(tO + 32u * q, o);
                        tmem_ld_wait();
                        tmem_pin(o);
#pragma unroll
                        for (int c = 0; c < 32; c++) o[c] = __float_as_uint(__uint_as_float(o[c]) * a);
                        tmem_st32(tO + 32u * q, o);
                    }
                }
                float y0 = 0.f, y1 = 0.f;
#pragma unroll
                for (int w = 0; w < 32; w++) {
                    const float p0 = ex2(fmaf(__uint_as_float(u[2 * w]), sl2, -off));
                    const float p1 = ex2(fmaf(__uint_as_float(u[2 * w + 1]), sl2, -off));
                    y0 += p0;
                    y1 += p1;
                    pw[w] = pack_bf16x2(p0, p1);
                }
                l = fmaf(l, a, y0 + y1);
            } else {
#pragma unroll
                for (int w = 0; w < 32; w++) pw[w] = 0u;
            }
            tmem_st32(tP, pw);
            tmem_st_wait();
            tc_fence_before();
            mbar_arrive(b_p + 8 * bsel);
        }
        if (ok && nent > 0) ok = __all_sync(0xffffffffu, mbar_wait(b_o, 0, ctl));
        tc_fence_after();
        if (ok) {
            const int qt = half ? qt1 : qt0;
            int token = -1;
            if (qt < p.nt) token = p.slot_src[qt * TE + (row & 63)];
            const bool live = token >= 0;
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const size_t orow = ((size_t)bh * p.seq + (live ? token : 0)) * kD;
            const float* co = p.coarse + ((size_t)bh * p.nt + min(qt, p.nt - 1)) * kD;
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
                    float g0 = 1.f, g1 = 1.f, g2 = 1.f, g3 = 1.f;
                    if (p.gate) {
                        const uint2 gw = *reinterpret_cast<const uint2*>(p.gate + orow + 32 * q + 4 * c);
                        g0 = __uint_as_float(gw.x << 16);
                        g1 = __uint_as_float(gw.x & 0xffff0000u);
                        g2 = __uint_as_float(gw.y << 16);
                        g3 = __uint_as_float(gw.y & 0xffff0000u);
                    }
                    f[4 * c] = __fadd_rn(__fmul_rn(cv.x, g0), __uint_as_float(o[4 * c]) * inv);
                    f[4 * c + 1] = __fadd_rn(__fmul_rn(cv.y, g1), __uint_as_float(o[4 * c + 1]) * inv);
                    f[4 * c + 2] = __fadd_rn(__fmul_rn(cv.z, g2), __uint_as_float(o[4 * c + 2]) * inv);
                    f[4 * c + 3] = __fadd_rn(__fmul_rn(cv.w, g3), __uint_as_float(o[4 * c + 3]) * inv);
                }
                if (p.out_is_bf16) {
                    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<unsigned short*>(p.out) + orow + 32 * q);
#pragma unroll
                    for (int c = 0; c < 4; c++)
                        dst[c] = make_uint4(pack_bf16x2(f[8 * c], f[8 * c + 1]), pack_bf16x2(f[8 * c + 2], f[8 * c + 3]),
                                            pack_bf16x2(f[8 * c + 4], f[8 * c + 5]), pack_bf16x2(f[8 * c + 6], f[8 * c + 7]));
                } else {
                    float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + orow + 32 * q);
#pragma unroll
                    for (int c = 0; c < 8; c++) dst[c] = make_float4(f[4 * c], f[4 * c + 1], f[4 * c + 2], f[4 * c + 3]);
                }
            }
        }
        tc_fence_before();
        asm volatile("bar.arrive 1, 160;" ::: "memory");
        return;
    }
    if (warp == 4) {
        // ------------------------------------------------------- TMA producer
        if (lane == 0) {
            WaitCtl ctl{abort_ptr, p.status, 11};
            tma_prefetch_desc(&tk);
            tma_prefetch_desc(&tv);
            int idx = 0;
            bool ok = true;
            // Ring order = consumption order: K0 K1 V0 K2 V1 K3 ... (Q.K^T runs two steps ahead of P.V)
            auto load = [&](int j, bool is_v) {
                if (!ok) return;
                const int tile = (int)(list[j] & 0xFFFFFu);
                const int slot = idx % kFineNS, use = idx / kFineNS;
                if (use > 0 && !mbar_wait(b_empty + 8 * slot, (use - 1) & 1, ctl)) { ok = false; return; }
                const uint32_t dst = ring + slot * kKvTileB, bar = b_full + 8 * slot;
                const CUtensorMap* map = is_v ? &tv : &tk;
                mbar_expect_tx(bar, kKvTileB);
                tma_load4(dst, map, bar, 0, tile * TE, bh, 0);
                tma_load4(dst + kKvPanelB, map, bar, 64, tile * TE, bh, 0);
                idx++;
            };
            if (nent > 0) load(0, false);
            if (nent > 1) load(1, false);
#pragma unroll 1
            for (int j = 0; j < nent && ok; j++) {
                load(j, true);
                if (j + 2 < nent) load(j + 2, false);
            }
            mbar_wait(b_q, 0, ctl);
            for (int s = 0; s < kFineNS && s < idx; s++) {
                const int last = ((idx - 1 - s) / kFineNS) * kFineNS + s;
                mbar_wait(b_full + 8 * s, (last / kFineNS) & 1, ctl);
            }
        }
        return;
    }
    // --------------------------------------------------------- MMA issuer (warp 5)
    if (lane == 0) {
        WaitCtl ctl{abort_ptr, p.status, 12};
        constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 64, 0);
        constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128, 1);
        bool ok = mbar_wait(b_q, 0, ctl);
        tc_fence_after();
        // ring index of K_j and V_j in the producer's order K0 K1 V0 K2 V1 ... V_{n-2} V_{n-1}
        auto idx_k = [&](int j) { return j < 2 ? j : 2 * j - 1; };
        auto idx_v = [&](int j) { return j == nent - 1 ? 2 * nent - 1 : 2 * j + 2; };
        const uint64_t a0 = umma_desc_sw128(sQ, 16, 1024);
        // S buffer (j & 1) = Q . K_j^T, then release K_j's slot
        auto qk = [&](int j) -> bool {
            const int ik = idx_k(j), slot = ik % kFineNS;
            if (!mbar_wait(b_full + 8 * slot, (ik / kFineNS) & 1, ctl)) return false;
            tc_fence_after();
            const uint64_t b0 = umma_desc_sw128(ring + slot * kKvTileB, 16, 1024);
            asm volatile(
                "{\n\t.reg .pred pt, pf;\n\t.reg .b64 a, b;\n\t"
                "setp.ne.b32 pf, %3, %3;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pf;\n\t"
                "add.s64 a, %1, 2;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
                "add.s64 a, %1, 4;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
                "add.s64 a, %1, 6;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
                "add.s64 a, %1, 1024;\n\tadd.s64 b, %2, 512;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
                "add.s64 a, %1, 1026;\n\tadd.s64 b, %2, 514;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
                "add.s64 a, %1, 1028;\n\tadd.s64 b, %2, 516;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
                "add.s64 a, %1, 1030;\n\tadd.s64 b, %2, 518;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, pt;\n\t"
                "}"
                ::"r"(tbase + 64u * (uint32_t)(j & 1)), "l"(a0), "l"(b0), "r"(idesc_qk)
                : "memory");
            umma_commit(b_s + 8 * (j & 1));
            umma_commit(b_empty + 8 * slot);
            return true;
        };
        if (ok && nent > 0) ok = qk(0);
        if (ok && nent > 1) ok = qk(1);
#pragma unroll 1
        for (int j = 0; j < nent && ok; j++) {
            const int iv = idx_v(j), slotV = iv % kFineNS;
            if (!mbar_wait(b_full + 8 * slotV, (iv / kFineNS) & 1, ctl)) { ok = false; break; }
            if (!mbar_wait(b_p + 8 * (j & 1), (j >> 1) & 1, ctl)) { ok = false; break; }
            tc_fence_after();
            {
                const uint64_t b0 = umma_desc_sw128(ring + slotV * kKvTileB, kKvPanelB, 1024);
                asm volatile(
                    "{\n\t.reg .pred pt, p0;\n\t.reg .b64 b;\n\t.reg .b32 t;\n\t"
                    "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 pt, %3, %3;\n\t"
                    "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
                    "add.u32 t, %1, 8;\n\tadd.s64 b, %2, 128;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
                    "add.u32 t, %1, 16;\n\tadd.s64 b, %2, 256;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
                    "add.u32 t, %1, 24;\n\tadd.s64 b, %2, 384;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [t], b, %3, pt;\n\t"
                    "}"
                    ::"r"(tbase + 128u), "r"(tbase + 64u * (uint32_t)(j & 1)), "l"(b0), "r"(idesc_pv), "r"((uint32_t)(j > 0))
                    : "memory");
            }
            umma_commit(b_od);
            umma_commit(b_empty + 8 * slotV);
            if (j == nent - 1) umma_commit(b_o);
            if (j + 2 < nent) ok = qk(j + 2);  // into the buffer P.V_j just read (same thread: in order)
        }
        umma_commit(b_drain);
        mbar_wait(b_drain, 0, ctl);
    }
    __syncwarp();
    asm volatile("bar.sync 1, 160;" ::: "memory");
    tc_fence_after();
    tmem_dealloc(tbase, 256);
#endif
}

static void host_tile_plan(Plan& pl) {
    const int t = pl.gt, h = pl.gh, w = pl.gw;
    const int nt = (t + 3) / 4, nh = (h + 3) / 4, nw = (w + 3) / 4;
    pl.nt = nt * nh * nw;
    pl.seq = t * h * w;
    pl.padded = pl.nt * TE;
    pl.slot_src.assign(pl.padded, -1);
    pl.token_slot.assign(pl.seq, 0);
    pl.block_sizes.assign(pl.nt, 0);
    int tile = 0;
    for (int tt = 0; tt < nt; tt++)
        for (int hh = 0; hh < nh; hh++)
            for (int ww = 0; ww < nw; ww++, tile++) {
                int slot = tile * TE;
                for (int z = tt * 4; z < std::min(tt * 4 + 4, t); z++)
                    for (int y = hh * 4; y < std::min(hh * 4 + 4, h); y++)
                        for (int x = ww * 4; x < std::min(ww * 4 + 4, w); x++) {
                            const int token = (z * h + y) * w + x;
                            pl.slot_src[slot] = token;
                            pl.token_slot[token] = (uint32_t)slot;
                            slot++;
                        }
                pl.block_sizes[tile] = (uint32_t)(slot - tile * TE);
            }
}

struct Workspace {
    __nv_bfloat16 *qt, *kt, *vt;
    float *means, *scores, *coarse;
    uint32_t* selected;
    size_t bytes;
};
static Workspace carve(void* base, int bh, int nt, int topk) {
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    Workspace w{};
    size_t o = 0;
    char* b = (char*)base;
    const size_t tiled = up((size_t)bh * nt * TE * kD * 2);
    w.qt = (__nv_bfloat16*)(b + o); o += tiled;
    w.kt = (__nv_bfloat16*)(b + o); o += tiled;
    w.vt = (__nv_bfloat16*)(b + o); o += tiled;
    w.means = (float*)(b + o); o += up((size_t)3 * bh * nt * kD * 4);
    w.scores = (float*)(b + o); o += up((size_t)bh * nt * nt * 4);
    w.coarse = (float*)(b + o); o += up((size_t)bh * nt * kD * 4);
    w.selected = (uint32_t*)(b + o); o += up((size_t)bh * nt * topk * 4);
    w.bytes = o;
    return w;
}

}  // namespace fvvsa

using fvvsa::Plan;

extern "C" int fv_vsa_topk_for(double sparsity, int num_tiles) {
    long long keep = (long long)ceil((1.0 - sparsity) * (double)num_tiles);
    const long long hi = std::max(num_tiles, 1);
    return (int)std::min(std::max(keep, 1ll), hi);
}

extern "C" int fv_vsa_plan_create(int gt, int gh, int gw, void** plan_out) {
    fvrt::clear_error();
    if (!plan_out) return fvrt::fail(FV_ERR_INVALID, "vsa: null plan_out");
    if (gt <= 0 || gh <= 0 || gw <= 0) return fvrt::fail(FV_ERR_INVALID, "vsa: empty grid (%d, %d, %d)", gt, gh, gw);
    if ((long long)gt * gh * gw > 0x3fffffffll) return FV_DECLINED;
    Plan* pl = new Plan();
    pl->gt = gt; pl->gh = gh; pl->gw = gw;
    pl->device = -1;
    pl->d_slot_src = nullptr;
    pl->d_block_sizes = nullptr;
    fvvsa::host_tile_plan(*pl);
    *plan_out = pl;
    return FV_RAN;
}
extern "C" int fv_vsa_plan_destroy(void* plan) {
    fvrt::clear_error();
    Plan* pl = (Plan*)plan;
    if (!pl) return FV_RAN;
    if (pl->d_slot_src) cudaFree(pl->d_slot_src);
    if (pl->d_block_sizes) cudaFree(pl->d_block_sizes);
    delete pl;
    return FV_RAN;
}
extern "C" int fv_vsa_plan_info(void* plan, int* num_tiles, int* seq, int* padded, int tiles[3]) {
    Plan* pl = (Plan*)plan;
    if (!pl) return fvrt::fail(FV_ERR_INVALID, "vsa: null plan");
    if (num_tiles) *num_tiles = pl->nt;
    if (seq) *seq = pl->seq;
    if (padded) *padded = pl->padded;
    if (tiles) { tiles[0] = (pl->gt + 3) / 4; tiles[1] = (pl->gh + 3) / 4; tiles[2] = (pl->gw + 3) / 4; }
    return FV_RAN;
}
extern "C" int fv_vsa_plan_host(void* plan, int32_t* slot_src, uint32_t* token_slot, uint32_t* block_sizes) {
    Plan* pl = (Plan*)plan;
    if (!pl) return fvrt::fail(FV_ERR_INVALID, "vsa: null plan");
    if (slot_src) memcpy(slot_src, pl->slot_src.data(), pl->slot_src.size() * 4);
    if (token_slot) memcpy(token_slot, pl->token_slot.data(), pl->token_slot.size() * 4);
    if (block_sizes) memcpy(block_sizes, pl->block_sizes.data(), pl->block_sizes.size() * 4);
    return FV_RAN;
}
extern "C" size_t fv_vsa_workspace_bytes(void* plan, int bh, int topk) {
    Plan* pl = (Plan*)plan;
    if (!pl || bh <= 0 || topk <= 0) return 0;
    return fvvsa::carve(nullptr, bh, pl->nt, std::min(topk, pl->nt)).bytes;
}

static int plan_upload(Plan* pl, int dev) {
    if (pl->device == dev && pl->d_slot_src) return FV_RAN;
    if (pl->d_slot_src) { cudaFree(pl->d_slot_src); cudaFree(pl->d_block_sizes); }
    FV_CUDA(cudaMalloc(&pl->d_slot_src, pl->slot_src.size() * 4));
    FV_CUDA(cudaMalloc(&pl->d_block_sizes, pl->block_sizes.size() * 4));
    FV_CUDA(cudaMemcpy(pl->d_slot_src, pl->slot_src.data(), pl->slot_src.size() * 4, cudaMemcpyHostToDevice));
    FV_CUDA(cudaMemcpy(pl->d_block_sizes, pl->block_sizes.data(), pl->block_sizes.size() * 4, cudaMemcpyHostToDevice));
    pl->device = dev;
    return FV_RAN;
}

extern "C" int fv_vsa_plan_upload(void* plan) {
    fvrt::clear_error();
    Plan* pl = (Plan*)plan;
    if (!pl) return fvrt::fail(FV_ERR_INVALID, "vsa: null plan");
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    return plan_upload(pl, dev);
}

extern "C" int fv_vsa_forward_bf16(void* stream_, void* plan, const void* q, const void* k, const void* v, const void* gate,
                                   int bh, int topk, float scale, void* out, int out_is_bf16, void* workspace,
                                   size_t workspace_bytes, uint32_t* selected_out, float* scores_out, float* coarse_out) {
    fvrt::clear_error();
    Plan* pl = (Plan*)plan;
    if (!pl) return fvrt::fail(FV_ERR_INVALID, "vsa: null plan");
    if (bh <= 0 || bh > 65535) return FV_DECLINED;  // bh rides in grid.y / grid.z of the small kernels
    if (pl->nt > 4096 || pl->nt >= (1 << 20)) return FV_DECLINED;  // the selection kernel keeps a row in shared memory
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (!q || !k || !v || !out || !workspace) return fvrt::fail(FV_ERR_INVALID, "vsa: null operand");
    if (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)out | (uintptr_t)gate | (uintptr_t)workspace) & 15)
        return fvrt::fail(FV_ERR_INVALID, "vsa: operands must be 16-byte aligned");
    if (!(scale > 0.f) || !isfinite(scale)) return fvrt::fail(FV_ERR_INVALID, "vsa: scale must be positive and finite");
    const int nt = pl->nt, seq = pl->seq;
    topk = std::min(std::max(topk, 1), nt);
    const fvvsa::Workspace w = fvvsa::carve(workspace, bh, nt, topk);
    if (workspace_bytes < w.bytes)
        return fvrt::fail(FV_ERR_INVALID, "vsa: workspace holds %zu bytes, %zu needed", workspace_bytes, w.bytes);
    rc = plan_upload(pl, dev);
    if (rc != FV_RAN) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    using bf = __nv_bfloat16;

    fvvsa::vsa_prep_kernel<<<dim3(nt, bh), 192, 0, stream>>>((const bf*)q, (const bf*)k, (const bf*)v, pl->d_slot_src,
                                                             pl->d_block_sizes, seq, nt, w.qt, w.kt, w.vt, w.means);
    FV_CUDA(cudaGetLastError());
    const float* qc = w.means;
    const float* kc = w.means + (size_t)bh * nt * fvvsa::kD;
    const float* vc = w.means + (size_t)2 * bh * nt * fvvsa::kD;
    {
        static bool score_attr[64] = {};
        if (!score_attr[dev]) {
            FV_CUDA(cudaFuncSetAttribute(fvvsa::vsa_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fvvsa::kScoreSmem));
            score_attr[dev] = true;
        }
        const int nb = (nt + fvvsa::kScoreTile - 1) / fvvsa::kScoreTile;
        fvvsa::vsa_scores_kernel<<<dim3(nb, nb, bh), 256, fvvsa::kScoreSmem, stream>>>(qc, kc, nt, scale, w.scores);
    }
    FV_CUDA(cudaGetLastError());
    {
        const size_t csm = (size_t)nt * sizeof(double) + (size_t)fvvsa::kCoarseQT * nt * sizeof(float);
        static size_t coarse_attr[64] = {};
        if (csm > 48 * 1024 && coarse_attr[dev] < csm) {
            FV_CUDA(cudaFuncSetAttribute(fvvsa::vsa_coarse_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csm));
            coarse_attr[dev] = csm;
        }
        fvvsa::vsa_coarse_kernel<<<dim3((nt + fvvsa::kCoarseQT - 1) / fvvsa::kCoarseQT, bh), 128, csm, stream>>>(w.scores, vc, nt,
                                                                                                            w.coarse);
    }
    FV_CUDA(cudaGetLastError());
    if (nt <= fvvsa::kTopkWarpMax) {
        const long long rows = (long long)bh * nt;
        fvvsa::vsa_topk_warp_kernel<<<(unsigned)((rows + 7) / 8), 256, (size_t)8 * nt * sizeof(uint32_t), stream>>>(
            w.scores, (int)rows, nt, topk, w.selected);
    } else {
        fvvsa::vsa_topk_kernel<<<dim3(nt, bh), 256, (size_t)nt * sizeof(uint32_t), stream>>>(w.scores, nt, topk, w.selected);
    }
    FV_CUDA(cudaGetLastError());

    fvvsa::FineParams fp{};
    fp.selected = w.selected;
    fp.block_sizes = pl->d_block_sizes;
    fp.slot_src = pl->d_slot_src;
    fp.coarse = w.coarse;
    fp.gate = (const bf*)gate;
    fp.out = out;
    fp.out_is_bf16 = out_is_bf16 ? 1 : 0;
    fp.bh = bh;
    fp.nt = nt;
    fp.topk = topk;
    fp.seq = seq;
    fp.sl2 = scale * 1.4426950408889634f;
    fp.list_cap = std::min(2 * topk, nt);
    rc = fvrt::status_word(dev, &fp.status);
    if (rc != FV_RAN) return rc;
    // shared memory: fixed part + union list + the two staged selections behind it
    const size_t smem = 1024 + fvvsa::kQTileB + fvvsa::kFineNS * fvvsa::kKvTileB + 256 + 4 * ((size_t)fp.list_cap + 2 * (size_t)topk);
    if (smem > 232448) return FV_DECLINED;
    CUtensorMap tq, tk, tv;
    const uint64_t dims[4] = {128, (uint64_t)nt * fvvsa::TE, (uint64_t)bh, 1};
    const uint64_t str[3] = {256, (uint64_t)nt * fvvsa::TE * 256, (uint64_t)nt * fvvsa::TE * 256 * bh};
    if ((rc = fvrt::encode_map4(&tq, w.qt, dims, str, 128)) != FV_RAN) return rc;
    if ((rc = fvrt::encode_map4(&tk, w.kt, dims, str, 64)) != FV_RAN) return rc;
    if ((rc = fvrt::encode_map4(&tv, w.vt, dims, str, 64)) != FV_RAN) return rc;
    static size_t attr_smem[64] = {};
    if (attr_smem[dev] < smem) {
        FV_CUDA(cudaFuncSetAttribute(fvvsa::fv_vsa_fine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_smem[dev] = smem;
    }
    const long long grid = (long long)((nt + 1) / 2) * bh;
    if (grid > 0x7fffffffll) return FV_DECLINED;
    fvvsa::fv_vsa_fine_kernel<<<(unsigned)grid, fvvsa::kFineThreads, smem, stream>>>(tq, tk, tv, fp);
    FV_CUDA(cudaGetLastError());
    if (selected_out)
        FV_CUDA(cudaMemcpyAsync(selected_out, w.selected, (size_t)bh * nt * topk * 4, cudaMemcpyDeviceToDevice, stream));
    if (scores_out)
        FV_CUDA(cudaMemcpyAsync(scores_out, w.scores, (size_t)bh * nt * nt * 4, cudaMemcpyDeviceToDevice, stream));
    if (coarse_out)
        FV_CUDA(cudaMemcpyAsync(coarse_out, w.coarse, (size_t)bh * nt * fvvsa::kD * 4, cudaMemcpyDeviceToDevice, stream));
    return FV_RAN;
}

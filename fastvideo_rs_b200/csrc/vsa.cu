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
// fv_vsa_fine_kernel: vsa_fine.cuh (included below, after this namespace's small kernels).

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

#include "vsa_fine.cuh"

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

    fvvsa::FineJob fp{};
    fp.selected = w.selected;
    fp.block_sizes = pl->d_block_sizes;
    fp.slot_src = pl->d_slot_src;
    fp.coarse = w.coarse;
    fp.gate = (const bf*)gate;
    fp.out = out;
    fp.out_is_bf16 = out_is_bf16 ? 1 : 0;
    fp.planes = bh;
    fp.tiles = nt;
    fp.topk = topk;
    fp.seq = seq;
    fp.sl2 = scale * 1.4426950408889634f;
    fp.list_cap = std::min(2 * topk, nt);
    rc = fvrt::status_word(dev, &fp.status);
    if (rc != FV_RAN) return rc;
    // shared memory: fixed part + union list + the two staged selections behind it
    const size_t smem = fvvsa::FineSmem::bytes(fp.list_cap, topk);
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

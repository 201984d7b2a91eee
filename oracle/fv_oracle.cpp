// TEST INFRASTRUCTURE, NOT PRODUCT: a CPU restatement of the reference's host
// math for the Wan self-attention path (zaitrarrio/fastvideo-rs; the reference
// is Rust and no Rust toolchain exists where this is built).  Only tests,
// the smoke check and the bench's CPU-baseline leg may load it; the library
// under test never does.
//
// Every function names the reference lines it restates (paths inside that
// repository, C/ = crates/fastvideo-cudarc/src/).  Arithmetic order follows
// the reference exactly: f32 with separate multiply and add (build with
// -ffp-contract=off), sequential sums, f64 only where the reference says f64.
// Known deviation: Rust's f32::exp / f64::exp / cos / sin call the platform
// libm, as glibc does here; results may differ from another libm in the last
// ulp.
//
// Parity pin: the reference holds no golden tensors for this path (its tests
// compare two implementations at run time); the closed-form unit tests it
// does have (C/rt/vsa.rs:481-695, C/rt/sp.rs:66-84, C/rt/attn.rs:883-930,
// C/rt/sdpa.rs:513-542) are re-run against this file by tests/test_oracle_*.py.
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <vector>

#include <atomic>
#include <thread>

#define FVO_API extern "C" __attribute__((visibility("default")))

// Host threads: FVO_THREADS, else every hardware thread.  (The reference's host ops use rayon
// over the same independent units: one (batch, head) plane or one row per task.)
static int fvo_threads() {
    const char* e = getenv("FVO_THREADS");
    int n = e ? atoi(e) : 0;
    if (n <= 0) n = (int)std::thread::hardware_concurrency();
    return n > 0 ? n : 1;
}
// Dynamic chunks of `grain` consecutive indices per grab; fn(worker_state, index).
template <class Make, class Fn>
static void parallel_for(long long n, long long grain, Make make, Fn fn) {
    const int nt = (int)std::min<long long>(fvo_threads(), std::max<long long>(1, (n + grain - 1) / grain));
    std::atomic<long long> next(0);
    auto body = [&]() {
        auto st = make();
        for (;;) {
            const long long b = next.fetch_add(grain);
            if (b >= n) break;
            const long long e = std::min(n, b + grain);
            for (long long i = b; i < e; i++) fn(st, i);
        }
    };
    if (nt <= 1) {
        body();
        return;
    }
    std::vector<std::thread> th;
    for (int i = 1; i < nt; i++) th.emplace_back(body);
    body();
    for (auto& t : th) t.join();
}

// ---- bf16 round to nearest even, NaN kept quiet --------------------------------
// C/rt/kernels/core.cu:2-15 (== half::bf16::from_f32, C/rt/ops.rs:1654-1656)
static inline uint16_t bf16_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static inline float bf16_val(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
FVO_API void fvo_bf16_round(const float* x, float* y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = bf16_val(bf16_bits(x[i]));
}
FVO_API void fvo_f32_to_bf16(const float* x, uint16_t* y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = bf16_bits(x[i]);
}
FVO_API void fvo_bf16_to_f32(const uint16_t* x, float* y, size_t n) {
    for (size_t i = 0; i < n; i++) y[i] = bf16_val(x[i]);
}

// ---- RoPE tables ----------------------------------------------------------------
// rotary_1d: C/wan/transformer.rs:447-463.  freq = (1 / theta^(2i/dim)) computed in
// f64 then narrowed to f32; arg = p (as f32) * freq in f32; cos/sin in f32; each
// value repeated twice (interleave).
static void rotary_1d(int dim, int seq, double theta, std::vector<float>& c, std::vector<float>& s) {
    const int half = dim / 2;
    c.assign((size_t)seq * dim, 0.f);
    s.assign((size_t)seq * dim, 0.f);
    for (int p = 0; p < seq; p++) {
        for (int i = 0; i < half; i++) {
            const float freq = (float)(1.0 / pow(theta, 2.0 * (double)i / (double)dim));
            const float arg = (float)p * freq;
            const float cv = cosf(arg), sv = sinf(arg);
            c[(size_t)p * dim + 2 * i] = cv;
            c[(size_t)p * dim + 2 * i + 1] = cv;
            s[(size_t)p * dim + 2 * i] = sv;
            s[(size_t)p * dim + 2 * i + 1] = sv;
        }
    }
}
// wan_rope_at: C/wan/transformer.rs:490-544.  Token grid (ppf, pph, ppw) already in
// patches; head dim d split t = d - 2*(2*(d/6)), h = w = 2*(d/6); row = [t | h | w];
// tokens ordered frame-major, then height, then width.  cos, sin: [ppf*pph*ppw, d].
FVO_API void fvo_wan_rope(int ppf, int pph, int ppw, int d, double theta, int start_frame, float* cos_out,
                          float* sin_out) {
    const int h_dim = 2 * (d / 6), w_dim = h_dim, t_dim = d - h_dim - w_dim;
    std::vector<float> ct, st, ch, sh, cw, sw;
    rotary_1d(t_dim, start_frame + ppf, theta, ct, st);
    rotary_1d(h_dim, pph, theta, ch, sh);
    rotary_1d(w_dim, ppw, theta, cw, sw);
    size_t o = 0;
    for (int ft = start_frame; ft < start_frame + ppf; ft++)
        for (int fh = 0; fh < pph; fh++)
            for (int fw = 0; fw < ppw; fw++) {
                memcpy(cos_out + o, &ct[(size_t)ft * t_dim], sizeof(float) * t_dim);
                memcpy(sin_out + o, &st[(size_t)ft * t_dim], sizeof(float) * t_dim);
                o += t_dim;
                memcpy(cos_out + o, &ch[(size_t)fh * h_dim], sizeof(float) * h_dim);
                memcpy(sin_out + o, &sh[(size_t)fh * h_dim], sizeof(float) * h_dim);
                o += h_dim;
                memcpy(cos_out + o, &cw[(size_t)fw * w_dim], sizeof(float) * w_dim);
                memcpy(sin_out + o, &sw[(size_t)fw * w_dim], sizeof(float) * w_dim);
                o += w_dim;
            }
}

// ---- q/k RMSNorm (+ RoPE) into BHSD ---------------------------------------------
// ops::host::qk_norm_rope_bhsd, C/rt/ops.rs:2304-2350.  The mean of squares runs over
// the full heads*d row (sequential f32 sum); inv = 1/sqrt(ms + eps); value =
// (x*inv)*w; pairs (even, even+1) rotate with cos[s, even] and sin[s, even+1].
// per_head != 0 switches the statistic to one head's d values (the reference's other
// scope, C/rt/fuse/policy.rs:414-424); w is then indexed the same way.
FVO_API void fvo_qk_norm_rope_bhsd(const float* src, const float* w, const float* cosv, const float* sinv, int batch,
                                   int seq, int heads, int d, int src_width, int col_off, float eps, int per_head,
                                   float* out) {
    const int width = heads * d;
    parallel_for(batch * heads, 1, [] { return 0; }, [&](int&, long long bhl) {
        const int bh = (int)bhl;
        const int b = bh / heads, h = bh % heads;
        float* plane = out + (size_t)bh * seq * d;
        for (int s = 0; s < seq; s++) {
            const float* x = src + ((size_t)b * seq + s) * src_width + col_off;
            float ss = 0.f;
            float ms;
            if (per_head) {
                for (int j = 0; j < d; j++) ss += x[h * d + j] * x[h * d + j];
                ms = ss / (float)d;
            } else {
                for (int j = 0; j < width; j++) ss += x[j] * x[j];
                ms = ss / (float)width;
            }
            const float inv = 1.0f / sqrtf(ms + eps);
            float* o = plane + (size_t)s * d;
            for (int p = 0; p < d; p++) {
                const int j = h * d + p;
                if (!cosv) {
                    o[p] = x[j] * inv * w[j];
                } else {
                    const int even = p - (p & 1);
                    const int j0 = h * d + even;
                    const float x1 = x[j0] * inv * w[j0];
                    const float x2 = x[j0 + 1] * inv * w[j0 + 1];
                    const float c = cosv[(size_t)s * d + even];
                    const float sn = sinv[(size_t)s * d + even + 1];
                    o[p] = (p & 1) ? (x1 * sn + x2 * c) : (x1 * c - x2 * sn);
                }
            }
        }
    });
}
// split_heads_bhsd: C/rt/ops.rs:2352-2371
FVO_API void fvo_split_heads_bhsd(const float* src, int batch, int seq, int heads, int d, int src_width, int col_off,
                                  float* out) {
    for (int bh = 0; bh < batch * heads; bh++) {
        const int b = bh / heads, h = bh % heads;
        for (int s = 0; s < seq; s++)
            memcpy(out + ((size_t)bh * seq + s) * d, src + ((size_t)b * seq + s) * src_width + col_off + h * d,
                   sizeof(float) * d);
    }
}

// ---- block-causal predicate --------------------------------------------------------
// BlockCausal::allows, C/rt/attn.rs:448-453
static inline bool bc_allows(int bt, int window, int sink, int q, int k) {
    if (bt < 1) bt = 1;
    const int tq = q / bt, tk = k / bt;
    return (tk <= tq && (window == 0 || tq - tk < window)) || tk < sink;
}
// BlockCausal::dense_mask, C/rt/attn.rs:455-466 (0 visible, -1e9 masked)
FVO_API void fvo_block_causal_mask(int bt, int window, int sink, int sq, int sk, float* mask) {
    for (int q = 0; q < sq; q++)
        for (int k = 0; k < sk; k++) mask[(size_t)q * sk + k] = bc_allows(bt, window, sink, q, k) ? 0.f : -1e9f;
}
// causal_temporal_mask, crates/fastvideo-models/src/wan/family.rs:80-109; local_attn_size < 0
// means no window.  frame_tokens = tokens per latent frame, frames_per_block >= 1.
FVO_API void fvo_causal_temporal_mask(int seq, int frame_tokens, int frames_per_block, int local_attn_size,
                                      float* mask) {
    const long long block = (long long)std::max(frames_per_block, 1) * frame_tokens;
    const long long blk = std::max<long long>(block, 1);
    for (int q = 0; q < seq; q++) {
        const long long end = ((long long)q / blk + 1) * block;
        for (int k = 0; k < seq; k++) {
            bool in_window = true;
            if (local_attn_size >= 0) in_window = (long long)k + (long long)local_attn_size * frame_tokens >= end;
            const bool ok = ((long long)k < end && in_window) || k == q;
            mask[(size_t)q * seq + k] = ok ? 0.f : -1e9f;
        }
    }
}

// ---- composed SDPA in f32 ------------------------------------------------------------
// sdpa_composed, C/rt/sdpa.rs:328-342: scores = (q @ k^T) * scale (+ mask); softmax; @ v.
// matmul order C/rt/tensor.rs:1688-1703: for each output row, for t in 0..k: row += a[i,t] * b[t,:]
// (f32, multiply then add).  softmax_last C/rt/ops.rs:2178-2193: m = max, e = exp(x - m) summed
// sequentially, inv = 1/sum, e *= inv.
// Evaluates only the query rows listed in `rows` (every row is independent); out is
// [bh, nrows, d].  mask: optional additive [sq, sk]; mask_mode 1 adds the block-causal mask
// (0 / -1e9) of (bt, window, sink) for global query index q_row0 + row instead.
FVO_API void fvo_sdpa_rows(const float* q, const float* k, const float* v, int bh, int sq, int sk, int d, float scale,
                           const float* mask, int mask_mode, int bt, int window, int sink, int q_row0, const int* rows,
                           int nrows, float* out) {
    // k^T once per head so the inner loop over keys is contiguous (same arithmetic).
    struct St {
        std::vector<float> kt, sc;
        int cur_h = -1;
    };
    const long long work = (long long)bh * nrows;
    parallel_for(work, 8, [&] { St st; st.kt.resize((size_t)d * sk); st.sc.resize(sk); return st; },
                 [&](St& st, long long wi) {
        const int h = (int)(wi / nrows), ri = (int)(wi % nrows);
        const int qi = rows[ri];
        std::vector<float>&kt = st.kt, &sc = st.sc;
        if (h != st.cur_h) {
            const float* kh = k + (size_t)h * sk * d;
            for (int j = 0; j < sk; j++)
                for (int t = 0; t < d; t++) kt[(size_t)t * sk + j] = kh[(size_t)j * d + t];
            st.cur_h = h;
        }
        const float* qr = q + ((size_t)h * sq + qi) * d;
        for (int j = 0; j < sk; j++) sc[j] = 0.f;
        for (int t = 0; t < d; t++) {
            const float av = qr[t];
            const float* kr = &kt[(size_t)t * sk];
            for (int j = 0; j < sk; j++) sc[j] += av * kr[j];
        }
        for (int j = 0; j < sk; j++) sc[j] *= scale;
        if (mask) {
            const float* mr = mask + (size_t)qi * sk;
            for (int j = 0; j < sk; j++) sc[j] += mr[j];
        } else if (mask_mode == 1) {
            for (int j = 0; j < sk; j++) sc[j] += bc_allows(bt, window, sink, q_row0 + qi, j) ? 0.f : -1e9f;
        }
        float m = -INFINITY;
        for (int j = 0; j < sk; j++) m = fmaxf(m, sc[j]);
        float sum = 0.f;
        for (int j = 0; j < sk; j++) {
            sc[j] = expf(sc[j] - m);
            sum += sc[j];
        }
        const float inv = 1.0f / sum;
        for (int j = 0; j < sk; j++) sc[j] *= inv;
        float* o = out + ((size_t)h * nrows + ri) * d;
        for (int c = 0; c < d; c++) o[c] = 0.f;
        const float* vh = v + (size_t)h * sk * d;
        for (int t = 0; t < sk; t++) {
            const float av = sc[t];
            const float* vr = vh + (size_t)t * d;
            for (int c = 0; c < d; c++) o[c] += av * vr[c];
        }
    });
}

// f64 cross-check (crates/fastvideo-gpucheck/src/kernels.rs:156-186 ref_sdpa; masked form
// crates/fastvideo-gpucheck/src/kernels_wan.rs:29-72): same selection of rows.
FVO_API void fvo_sdpa_rows_f64(const float* q, const float* k, const float* v, int bh, int sq, int sk, int d,
                               float scale, int mask_mode, int bt, int window, int sink, int q_row0, const int* rows,
                               int nrows, double* out) {
    const long long work = (long long)bh * nrows;
    parallel_for(work, 8, [&] { return std::vector<double>(sk); }, [&](std::vector<double>& sc, long long wi) {
        const int h = (int)(wi / nrows), ri = (int)(wi % nrows);
        const int qi = rows[ri];
        const float* qr = q + ((size_t)h * sq + qi) * d;
        double m = -INFINITY;
        for (int j = 0; j < sk; j++) {
            if (mask_mode == 1 && !bc_allows(bt, window, sink, q_row0 + qi, j)) {
                sc[j] = -INFINITY;
                continue;
            }
            const float* kr = k + ((size_t)h * sk + j) * d;
            double dot = 0;
            for (int t = 0; t < d; t++) dot += (double)qr[t] * (double)kr[t];
            sc[j] = dot * (double)scale;
            m = std::max(m, sc[j]);
        }
        double* o = out + ((size_t)h * nrows + ri) * d;
        for (int c = 0; c < d; c++) o[c] = 0;
        double z = 0;
        if (m > -INFINITY)
            for (int j = 0; j < sk; j++) {
                if (sc[j] == -INFINITY) continue;
                const double e = exp(sc[j] - m);
                z += e;
                const float* vr = v + ((size_t)h * sk + j) * d;
                for (int c = 0; c < d; c++) o[c] += e * (double)vr[c];
            }
        if (z > 0)
            for (int c = 0; c < d; c++) o[c] /= z;
    });
}

// ---- sequence-parallel split -----------------------------------------------------------
// sp::shard_ranges, C/rt/sp.rs:16-28: contiguous, remainder to the low ranks.
FVO_API void fvo_shard_ranges(int seq, int world, int* start, int* len) {
    if (world < 1) world = 1;
    const int base = seq / world, rem = seq % world;
    int s = 0;
    for (int r = 0; r < world; r++) {
        len[r] = base + (r < rem ? 1 : 0);
        start[r] = s;
        s += len[r];
    }
}

// f32::total_cmp as an integer key (IEEE totalOrder: -0 < +0, NaNs at the ends)
static inline int32_t total_key(float f) {
    int32_t b;
    memcpy(&b, &f, 4);
    return b ^ (int32_t)((uint32_t)(b >> 31) >> 1);
}

// ---- VSA ----------------------------------------------------------------------------------
// topk_for, C/rt/vsa.rs:34-37
FVO_API int fvo_topk_for(double sparsity, int num_tiles) {
    long long keep = (long long)ceil((1.0 - sparsity) * (double)num_tiles);
    const long long hi = std::max(num_tiles, 1);
    if (keep < 1) keep = 1;
    if (keep > hi) keep = hi;
    return (int)keep;
}
// TilePlan::new, C/rt/vsa.rs:63-108.  Tile = 4x4x4 cube, 64 slots.  Outputs sized by the caller:
// slot_src [ntiles*64] (-1 = padding), token_slot [t*h*w], block_sizes [ntiles].  Returns ntiles.
FVO_API int fvo_tile_plan(int t, int h, int w, int32_t* slot_src, uint32_t* token_slot, uint32_t* block_sizes) {
    const int ts = 4, hs = 4, ws = 4, TE = 64;
    const int nt = (t + ts - 1) / ts, nh = (h + hs - 1) / hs, nw = (w + ws - 1) / ws;
    const int ntiles = nt * nh * nw;
    if (!slot_src) return ntiles;
    for (int i = 0; i < ntiles * TE; i++) slot_src[i] = -1;
    int tile = 0;
    for (int tt = 0; tt < nt; tt++)
        for (int hh = 0; hh < nh; hh++)
            for (int ww = 0; ww < nw; ww++) {
                int slot = tile * TE;
                for (int z = tt * ts; z < std::min((tt + 1) * ts, t); z++)
                    for (int y = hh * hs; y < std::min((hh + 1) * hs, h); y++)
                        for (int x = ww * ws; x < std::min((ww + 1) * ws, w); x++) {
                            const int token = (z * h + y) * w + x;
                            slot_src[slot] = token;
                            token_slot[token] = (uint32_t)slot;
                            slot++;
                        }
                block_sizes[tile] = (uint32_t)(slot - tile * TE);
                tile++;
            }
    return ntiles;
}

// vsa_attention_host, C/rt/vsa.rs:116-262, as written: f32 tile means (in-order sum over the
// tile's real slots, then divide by the real count), f64 coarse dot * f64(scale) narrowed to f32,
// f64 softmax over tiles, coarse accumulated in f32 from f64 products, top-k by score descending
// with ties to the lower index, f64 fine attention with an online max in f32, out = coarse*gate +
// sparse.  q, k, v, gate, out: [b*heads, seq, dim] f32 (gate may be null = ones).
// Optional outputs: selected [b*heads, ntiles, topk] in the reference's emission order,
// scores [b*heads, ntiles, ntiles], coarse [b*heads, ntiles, dim].
FVO_API void fvo_vsa_attention_host(const float* q, const float* k, const float* v, const float* gate, int gt, int gh,
                                    int gw, int topk, int bheads, int dim, float scale, float* out,
                                    uint32_t* selected_out, float* scores_out, float* coarse_out) {
    const int TE = 64;
    const int seq = gt * gh * gw;
    const int nb = fvo_tile_plan(gt, gh, gw, nullptr, nullptr, nullptr);
    std::vector<int32_t> slot_src((size_t)nb * TE);
    std::vector<uint32_t> token_slot(seq), block_sizes(nb);
    fvo_tile_plan(gt, gh, gw, slot_src.data(), token_slot.data(), block_sizes.data());
    topk = std::min(std::max(topk, 1), nb);
    parallel_for(bheads, 1, [] { return 0; }, [&](int&, long long bhl) {
        const int bh = (int)bhl;
        const size_t base = (size_t)bh * seq * dim;
        std::vector<float> qc((size_t)nb * dim, 0.f), kc((size_t)nb * dim, 0.f), vc((size_t)nb * dim, 0.f);
        for (int tile = 0; tile < nb; tile++) {
            const float n = (float)block_sizes[tile];
            if (n == 0.f) continue;
            for (int slot = tile * TE; slot < tile * TE + (int)block_sizes[tile]; slot++) {
                const size_t token = (size_t)slot_src[slot];
                const float *qr = q + base + token * dim, *kr = k + base + token * dim, *vr = v + base + token * dim;
                for (int d = 0; d < dim; d++) {
                    qc[(size_t)tile * dim + d] += qr[d];
                    kc[(size_t)tile * dim + d] += kr[d];
                    vc[(size_t)tile * dim + d] += vr[d];
                }
            }
            for (int d = 0; d < dim; d++) {
                qc[(size_t)tile * dim + d] /= n;
                kc[(size_t)tile * dim + d] /= n;
                vc[(size_t)tile * dim + d] /= n;
            }
        }
        std::vector<float> coarse((size_t)nb * dim, 0.f), scores((size_t)nb * nb, 0.f);
        std::vector<double> exps(nb);
        for (int qt = 0; qt < nb; qt++) {
            float* s = &scores[(size_t)qt * nb];
            for (int kt = 0; kt < nb; kt++) {
                double dot = 0;
                for (int d = 0; d < dim; d++) dot += (double)qc[(size_t)qt * dim + d] * (double)kc[(size_t)kt * dim + d];
                s[kt] = (float)(dot * (double)scale);
            }
            float m = -INFINITY;
            for (int kt = 0; kt < nb; kt++) m = fmaxf(m, s[kt]);
            double z = 0;
            for (int kt = 0; kt < nb; kt++) {
                exps[kt] = exp((double)(s[kt] - m));
                z += exps[kt];
            }
            for (int kt = 0; kt < nb; kt++) {
                const double wgt = exps[kt] / z;
                for (int d = 0; d < dim; d++) coarse[(size_t)qt * dim + d] += (float)(wgt * (double)vc[(size_t)kt * dim + d]);
            }
        }
        std::vector<uint32_t> selected((size_t)nb * topk), order(nb);
        for (int qt = 0; qt < nb; qt++) {
            const float* s = &scores[(size_t)qt * nb];
            for (int i = 0; i < nb; i++) order[i] = (uint32_t)i;
            // f32::total_cmp descending, then index ascending (stable sort of an ascending list)
            std::stable_sort(order.begin(), order.end(),
                             [&](uint32_t a, uint32_t b) { return total_key(s[a]) > total_key(s[b]); });
            for (int i = 0; i < topk; i++) selected[(size_t)qt * topk + i] = order[i];
        }
        for (int qt = 0; qt < nb; qt++) {
            const uint32_t* picks = &selected[(size_t)qt * topk];
            std::vector<double> acc(dim);
            for (int qslot = qt * TE; qslot < qt * TE + (int)block_sizes[qt]; qslot++) {
                const size_t qtok = (size_t)slot_src[qslot];
                const float* qr = q + base + qtok * dim;
                float m = -INFINITY;
                std::fill(acc.begin(), acc.end(), 0.0);
                double z = 0;
                for (int pi = 0; pi < topk; pi++) {
                    const int kt = (int)picks[pi];
                    for (int kslot = kt * TE; kslot < kt * TE + (int)block_sizes[kt]; kslot++) {
                        const size_t ktok = (size_t)slot_src[kslot];
                        const float* kr = k + base + ktok * dim;
                        double dot = 0;
                        for (int d = 0; d < dim; d++) dot += (double)qr[d] * (double)kr[d];
                        const float s = (float)(dot * (double)scale);
                        if (s > m) {
                            const double shrink = isfinite(m) ? exp((double)(m - s)) : 0.0;
                            z *= shrink;
                            for (int d = 0; d < dim; d++) acc[d] *= shrink;
                            m = s;
                        }
                        const double e = exp((double)(s - m));
                        z += e;
                        const float* vr = v + base + ktok * dim;
                        for (int d = 0; d < dim; d++) acc[d] += e * (double)vr[d];
                    }
                }
                const size_t dst = base + qtok * dim;
                for (int d = 0; d < dim; d++) {
                    const float sparse = z > 0.0 ? (float)(acc[d] / z) : 0.f;
                    const float c = coarse[(size_t)qt * dim + d] * (gate ? gate[dst + d] : 1.0f);
                    out[dst + d] = c + sparse;
                }
            }
        }
        if (selected_out) memcpy(selected_out + (size_t)bh * nb * topk, selected.data(), sizeof(uint32_t) * nb * topk);
        if (scores_out) memcpy(scores_out + (size_t)bh * nb * nb, scores.data(), sizeof(float) * nb * nb);
        if (coarse_out) memcpy(coarse_out + (size_t)bh * nb * dim, coarse.data(), sizeof(float) * nb * dim);
    });
}

FVO_API int fvo_num_threads(void) { return fvo_threads(); }

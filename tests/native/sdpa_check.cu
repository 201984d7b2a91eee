// Standalone bring-up checker for libfvsdpa.so: runs fv_sdpa_dense_bf16 on a
// list of shapes, checks sampled rows against an f64 host evaluation of the
// same bf16 inputs, and times each case with CUDA events.  No torch, no
// Python: it exists so that a kernel change can be checked in seconds.
//
//   sdpa_check [--bench] [--selftest] [--trace STEPS] [--case bh,sq,sk[,block_tokens,window,sink]]...
//
// --trace STEPS: with a library built with -DFV_ATT_TRACE (a bring-up build, never the shipped one) every case
// is launched three times and the SM-clock stamps CTA 0 wrote during the last launch are printed, one line per
// role (smA / smB: lane 0 of the first softmax warp of row tile A / B; iss: the issuer) and key step:
//   smA/smB  0 S complete seen, 1 first 32 columns loaded, 2 exponentials done, 6 P handed over; on the last
//            step of an item also 3 last product seen, 4 / 5 first / second 32 columns of the output stored,
//            7 output stored
//   iss      0 K/V pair arrived, 2 / 5 P of tile A / B seen, 3 / 6 Q.K^T of tile A / B issued
// (cycles since the first stamp, -1 = not stamped).  Without such a build the option reports that and fails.
//
// --selftest also drives the bounded-wait failure path (fv_selftest_wait_timeout) and checks that
// fv_device_status reports it once and that a normal case runs afterwards.
//
// Exit code 0 when every case is within tolerance (max-abs 2e-2, mean-abs
// 2e-3 against the f64 evaluation) and no kernel reported a status.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <vector>
#include "../../include/fv_sdpa.h"

static uint16_t f2bf(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}
static float bf2f(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 0x1234567ull) {}
    uint64_t next() {
        uint64_t z = (s += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uni() { return ((next() >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
    float normal() {
        const double u1 = uni(), u2 = uni();
        return (float)(sqrt(-2.0 * log(u1)) * cos(6.283185307179586 * u2));
    }
};

// N(0,1) rounded to bf16.  Large tensors draw from a table of 2^20 normals through a hashed index (a full
// Box-Muller stream for a billion elements would take minutes on one host thread).
static void fill_normal(std::vector<uint16_t>& x, Rng& r) {
    if (x.size() <= (1u << 22)) {
        for (auto& e : x) e = f2bf(r.normal());
        return;
    }
    std::vector<uint16_t> table(1u << 20);
    for (auto& e : table) e = f2bf(r.normal());
    uint64_t s = r.next() | 1ull;
    for (size_t i = 0; i < x.size(); i++) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        x[i] = table[(s >> 40) & ((1u << 20) - 1)];
    }
}

struct Case {
    int bh, sq, sk, bt, win, sink;
};

#define CK(x)                                                                          \
    do {                                                                               \
        cudaError_t e = (x);                                                           \
        if (e != cudaSuccess) {                                                        \
            printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e), __FILE__, __LINE__); \
            exit(2);                                                                   \
        }                                                                              \
    } while (0)

static bool allows(const Case& c, int q, int k) {
    if (c.bt <= 0) return true;
    const int tq = q / c.bt, tk = k / c.bt;
    return (tk <= tq && (c.win == 0 || tq - tk < c.win)) || tk < c.sink;
}

static int run_case(const Case& c, bool bench, int out_bf16) {
    const size_t nq = (size_t)c.bh * c.sq * 128, nk = (size_t)c.bh * c.sk * 128;
    std::vector<uint16_t> q(nq), k(nk), v(nk);
    Rng r(1000003ull * c.bh + 7919ull * c.sq + c.sk);
    fill_normal(q, r);
    fill_normal(k, r);
    fill_normal(v, r);
    void *dq, *dk, *dv, *dout;
    const size_t out_bytes = nq * (out_bf16 ? 2 : 4);
    CK(cudaMalloc(&dq, nq * 2));
    CK(cudaMalloc(&dk, nk * 2));
    CK(cudaMalloc(&dv, nk * 2));
    CK(cudaMalloc(&dout, out_bytes));
    CK(cudaMemcpy(dq, q.data(), nq * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dk, k.data(), nk * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv, v.data(), nk * 2, cudaMemcpyHostToDevice));
    CK(cudaMemset(dout, 0xff, out_bytes));
    const float scale = 1.0f / sqrtf(128.f);
    const int mode = c.bt > 0 ? FV_MASK_BLOCK_CAUSAL : FV_MASK_NONE;
    int rc = fv_sdpa_dense_bf16(nullptr, dq, dk, dv, dout, out_bf16, c.bh, c.sq, c.sk, 128, scale, mode, c.bt, c.win,
                                c.sink, 0);
    if (rc != FV_RAN) {
        printf("case bh=%d sq=%d sk=%d: rc=%d %s\n", c.bh, c.sq, c.sk, rc, fv_last_error());
        return 1;
    }
    CK(cudaDeviceSynchronize());
    int code = 0;
    rc = fv_device_status(nullptr, &code);
    if (rc != FV_RAN) {
        printf("case bh=%d sq=%d sk=%d: device status %d (%s)\n", c.bh, c.sq, c.sk, code, fv_last_error());
        return 1;
    }
    std::vector<uint8_t> out(out_bytes);
    CK(cudaMemcpy(out.data(), dout, out_bytes, cudaMemcpyDeviceToHost));
    auto outv = [&](size_t i) -> float {
        return out_bf16 ? bf2f(((uint16_t*)out.data())[i]) : ((float*)out.data())[i];
    };
    // sampled rows: first, last, tile edges, and a pseudo-random spread
    std::vector<int> rows;
    const int probes[] = {0, 1, 31, 32, 63, 64, 127, 128, 129, 255, 256, 257, 383, 384, 511, 512};
    for (int pr : probes)
        if (pr < c.sq) rows.push_back(pr);
    for (int i = 1; i <= 8; i++) rows.push_back(c.sq - i >= 0 ? c.sq - i : 0);
    Rng rr(99);
    const int extra = c.sq * (long long)c.sk > 4000000 ? 12 : 48;
    for (int i = 0; i < extra; i++) rows.push_back((int)(rr.next() % (uint64_t)c.sq));
    std::sort(rows.begin(), rows.end());
    rows.erase(std::unique(rows.begin(), rows.end()), rows.end());
    std::vector<int> heads = {0, c.bh - 1, c.bh / 2};
    std::sort(heads.begin(), heads.end());
    heads.erase(std::unique(heads.begin(), heads.end()), heads.end());
    double max_abs = 0, sum_abs = 0;
    size_t cnt = 0, nan_cnt = 0;
    std::vector<double> s(c.sk), acc(128);
    for (int h : heads) {
        for (int qi : rows) {
            const uint16_t* qr = &q[((size_t)h * c.sq + qi) * 128];
            double m = -INFINITY;
            for (int j = 0; j < c.sk; j++) {
                if (!allows(c, qi, j)) {
                    s[j] = -INFINITY;
                    continue;
                }
                const uint16_t* kr = &k[((size_t)h * c.sk + j) * 128];
                double d = 0;
                for (int t = 0; t < 128; t++) d += (double)bf2f(qr[t]) * (double)bf2f(kr[t]);
                s[j] = d * (double)scale;
                m = std::max(m, s[j]);
            }
            double z = 0;
            std::fill(acc.begin(), acc.end(), 0.0);
            if (m > -INFINITY) {
                for (int j = 0; j < c.sk; j++) {
                    if (s[j] == -INFINITY) continue;
                    const double e = exp(s[j] - m);
                    z += e;
                    const uint16_t* vr = &v[((size_t)h * c.sk + j) * 128];
                    for (int t = 0; t < 128; t++) acc[t] += e * (double)bf2f(vr[t]);
                }
            }
            for (int t = 0; t < 128; t++) {
                const double want = z > 0 ? acc[t] / z : 0.0;
                const float got = outv(((size_t)h * c.sq + qi) * 128 + t);
                if (!(got == got)) {
                    nan_cnt++;
                    continue;
                }
                const double e = fabs((double)got - want);
                max_abs = std::max(max_abs, e);
                sum_abs += e;
                cnt++;
            }
        }
    }
    // every output element must have been written (buffer was filled with 0xff = NaN pattern)
    size_t unwritten = 0;
    for (size_t i = 0; i < nq; i++) {
        const float g = outv(i);
        if (!(g == g)) unwritten++;
    }
    const double mean_abs = cnt ? sum_abs / cnt : 0;
    const bool pass = max_abs <= 2e-2 && mean_abs <= 2e-3 && nan_cnt == 0 && unwritten == 0;
    double ms = 0, tflops = 0;
    if (bench) {
        cudaEvent_t e0, e1;
        CK(cudaEventCreate(&e0));
        CK(cudaEventCreate(&e1));
        std::vector<float> t;
        for (int i = 0; i < 7; i++) {
            CK(cudaEventRecord(e0));
            fv_sdpa_dense_bf16(nullptr, dq, dk, dv, dout, out_bf16, c.bh, c.sq, c.sk, 128, scale, mode, c.bt, c.win, c.sink,
                               0);
            CK(cudaEventRecord(e1));
            CK(cudaEventSynchronize(e1));
            float x;
            CK(cudaEventElapsedTime(&x, e0, e1));
            if (i >= 2) t.push_back(x);
        }
        std::sort(t.begin(), t.end());
        ms = t[t.size() / 2];
        double vis = 0;
        if (c.bt <= 0) {
            vis = (double)c.sq * c.sk;
        } else {
            for (int qi = 0; qi < c.sq; qi += 1) {
                // block-causal without window/sink in the bench cases: keys < end of the row's block
                long long hi = std::min<long long>(c.sk, ((long long)(qi / c.bt) + 1) * c.bt);
                vis += (double)hi;
            }
        }
        tflops = 4.0 * c.bh * vis * 128 / (ms * 1e-3) / 1e12;
    }
    printf("{\"case\": \"bh%d sq%d sk%d bt%d w%d s%d %s\", \"max_abs\": %.3e, \"mean_abs\": %.3e, \"nan\": %zu, \"unwritten\": %zu, "
           "\"checked\": %zu, \"ms\": %.4f, \"tflops\": %.1f, \"pass\": %s}\n",
           c.bh, c.sq, c.sk, c.bt, c.win, c.sink, out_bf16 ? "bf16" : "f32", max_abs, mean_abs, nan_cnt, unwritten, cnt, ms,
           tflops, pass ? "true" : "false");
    fflush(stdout);
    cudaFree(dq);
    cudaFree(dk);
    cudaFree(dv);
    cudaFree(dout);
    return pass ? 0 : 1;
}

// The stamps of one launch of a bring-up build (see the header).
static int trace_case(const Case& c, int steps) {
    typedef void (*set_trace_fn)(unsigned long long*, int);
    set_trace_fn set_trace = (set_trace_fn)dlsym(RTLD_DEFAULT, "fv_debug_set_trace");
    if (!set_trace) {
        printf("--trace: this libfvsdpa.so was built without -DFV_ATT_TRACE\n");
        return 1;
    }
    const size_t nq = (size_t)c.bh * c.sq * 128, nk = (size_t)c.bh * c.sk * 128;
    Rng r(7);
    std::vector<uint16_t> q(nq), k(nk), v(nk);
    fill_normal(q, r);
    fill_normal(k, r);
    fill_normal(v, r);
    void *dq, *dk, *dv, *dout;
    unsigned long long* dtr;
    const size_t tn = (size_t)4 * steps * 8;
    CK(cudaMalloc(&dq, nq * 2));
    CK(cudaMalloc(&dk, nk * 2));
    CK(cudaMalloc(&dv, nk * 2));
    CK(cudaMalloc(&dout, nq * 2));
    CK(cudaMalloc(&dtr, tn * 8));
    CK(cudaMemcpy(dq, q.data(), nq * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dk, k.data(), nk * 2, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(dv, v.data(), nk * 2, cudaMemcpyHostToDevice));
    const float scale = 1.f / sqrtf(128.f);
    for (int rep = 0; rep < 3; rep++) {
        CK(cudaMemset(dtr, 0, tn * 8));
        set_trace(rep == 2 ? dtr : nullptr, steps);
        const int rc = fv_sdpa_dense_bf16(nullptr, dq, dk, dv, dout, 1, c.bh, c.sq, c.sk, 128, scale,
                                          c.bt > 0 ? FV_MASK_BLOCK_CAUSAL : FV_MASK_NONE, c.bt, c.win, c.sink, 0);
        if (rc != FV_RAN) {
            printf("--trace: rc=%d %s\n", rc, fv_last_error());
            return 1;
        }
        CK(cudaDeviceSynchronize());
    }
    set_trace(nullptr, 0);
    std::vector<unsigned long long> t(tn);
    CK(cudaMemcpy(t.data(), dtr, tn * 8, cudaMemcpyDeviceToHost));
    unsigned long long t0 = ~0ull;
    for (unsigned long long x : t)
        if (x && x < t0) t0 = x;
    const char* names[3] = {"smA", "smB", "iss"};
    printf("# trace bh%d sq%d sk%d bt%d: role step ev0 .. ev7\n", c.bh, c.sq, c.sk, c.bt);
    for (int s = 0; s < steps; s++)
        for (int role = 0; role < 3; role++) {
            printf("%s %3d:", names[role], s);
            for (int e = 0; e < 8; e++) {
                const unsigned long long x = t[((size_t)role * steps + s) * 8 + e];
                printf(" %8lld", x ? (long long)(x - t0) : -1ll);
            }
            printf("\n");
        }
    cudaFree(dq);
    cudaFree(dk);
    cudaFree(dv);
    cudaFree(dout);
    cudaFree(dtr);
    return 0;
}

static int selftest() {
    int rc = fv_selftest_wait_timeout(nullptr, 2000000);
    if (rc != FV_RAN) {
        printf("selftest: launch rc=%d %s\n", rc, fv_last_error());
        return 1;
    }
    CK(cudaDeviceSynchronize());
    int code = 0;
    rc = fv_device_status(nullptr, &code);
    if (rc != FV_ERR_DEVICE_STATUS || code != 109) {
        printf("selftest: expected FV_ERR_DEVICE_STATUS / 109, got rc=%d code=%d\n", rc, code);
        return 1;
    }
    rc = fv_device_status(nullptr, &code);
    if (rc != FV_RAN || code != 0) {
        printf("selftest: the status word was not cleared (rc=%d code=%d)\n", rc, code);
        return 1;
    }
    printf("{\"case\": \"selftest: a wait ran out, status 109 reported once\", \"pass\": true}\n");
    return run_case(Case{2, 300, 512, 0, 0, 0}, false, 1);
}

int main(int argc, char** argv) {
    bool bench = false, st = false;
    int trace_steps = 0;
    std::vector<Case> cases;
    for (int i = 1; i < argc; i++) {
        if (!strcmp(argv[i], "--bench")) bench = true;
        else if (!strcmp(argv[i], "--selftest")) st = true;
        else if (!strcmp(argv[i], "--trace") && i + 1 < argc) trace_steps = atoi(argv[++i]);
        else if (!strcmp(argv[i], "--case") && i + 1 < argc) {
            Case c{1, 1, 1, 0, 0, 0};
            sscanf(argv[++i], "%d,%d,%d,%d,%d,%d", &c.bh, &c.sq, &c.sk, &c.bt, &c.win, &c.sink);
            cases.push_back(c);
        }
    }
    if (cases.empty()) {
        const Case def[] = {{1, 1, 1, 0, 0, 0},     {2, 128, 128, 0, 0, 0},  {2, 256, 256, 0, 0, 0},  {3, 192, 192, 0, 0, 0},
                            {2, 63, 4097, 0, 0, 0}, {2, 130, 1, 0, 0, 0},    {2, 300, 512, 0, 0, 0},  {2, 1000, 333, 0, 0, 0},
                            {4, 1024, 1024, 0, 0, 0}, {2, 257, 640, 0, 0, 0}, {2, 2048, 2048, 0, 0, 0},
                            {2, 600, 600, 100, 0, 0}, {2, 600, 600, 100, 2, 1}, {2, 1000, 1000, 130, 0, 0},
                            {1, 24, 24, 5, 2, 1},   {2, 2340, 2340, 780, 0, 0},
                            // more work items than SMs: every CTA takes several, Q ring and barrier phases wrap
                            {160, 512, 384, 0, 0, 0}, {8, 8192, 1024, 0, 0, 0}, {40, 2000, 640, 0, 0, 0},
                            {12, 4680, 4680, 1560, 0, 0}, {24, 3000, 512, 0, 0, 0}, {300, 130, 257, 0, 0, 0},
                            {20, 2500, 2500, 600, 2, 1}};
        for (const Case& c : def) cases.push_back(c);
    }
    int bad = 0;
    if (trace_steps > 0) {
        for (const Case& c : cases) bad += trace_case(c, trace_steps);
        return bad ? 1 : 0;
    }
    for (const Case& c : cases) {
        bad += run_case(c, bench, 1);
    }
    // f32 output on one small case
    if (argc == 1) bad += run_case(Case{2, 300, 512, 0, 0, 0}, false, 0);
    if (st) bad += selftest();
    printf("%s (%d failing)\n", bad ? "FAIL" : "OK", bad);
    return bad ? 1 : 0;
}

// Sequence parallelism behind the C ABI: one handle per rank (one process or thread per GPU), contiguous
// token shards (sp::shard_ranges, crates/fastvideo-cudarc/src/rt/sp.rs:16-28), one exchange per call --
// an NCCL all-gather of the rank's bf16 K and V shards into this rank's own HBM on a high-priority stream --
// overlapped with attention over the local keys; the second pass merges the other ranks' keys by
// log-sum-exp.  Replaces dispatch_sharded_multi_gpu (crates/fastvideo-cudarc/src/rt/sdpa.rs:354-410), which
// replicates K/V on every rank and gathers the outputs through the host.
//
// NCCL is looked up at run time (dlopen of libnccl.so.2: the copy the host process already loaded, if any),
// so the library has no link-time dependency on it and loads on machines without NCCL.
#include "fv_runtime.h"
#include <cuda_bf16.h>
#include <dlfcn.h>
#include <stdlib.h>
#include <time.h>
#include <mutex>
#if __has_include(<nccl.h>)
#include <nccl.h>  // types only (ncclConfig_t for the non-blocking rendezvous); every call goes through dlsym
#define FV_HAVE_NCCL_H 1
#else
#define FV_HAVE_NCCL_H 0
#endif
#include <string.h>
#include <vector>

namespace fvsp {

constexpr int kD = 128;
constexpr int kMaxGroups = 8;

// The part of NCCL's public C interface used here (nccl.h): ncclUniqueId is 128 opaque bytes, ncclSuccess = 0,
// ncclBfloat16 = 9.
struct NcclId {
    char bytes[128];
};
constexpr int kNcclBf16 = 9;
struct Nccl {
    void* lib = nullptr;
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(void**, int, NcclId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    // optional (NCCL >= 2.14): the non-blocking rendezvous
    int (*CommInitRankConfig)(void**, int, NcclId, int, void*) = nullptr;
    int (*CommGetAsyncError)(void*, int*) = nullptr;
    int (*CommAbort)(void*) = nullptr;
};
static Nccl g_nccl;
static std::mutex g_nccl_mu;

static int load_nccl() {
    std::lock_guard<std::mutex> lk(g_nccl_mu);
    if (g_nccl.lib) return FV_RAN;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
    if (!h) return fvrt::fail(FV_ERR_NCCL, "libnccl.so.2 not found: %s", dlerror());
    Nccl n;
    n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    n.AllGather = reinterpret_cast<decltype(n.AllGather)>(dlsym(h, "ncclAllGather"));
    n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    n.CommInitRankConfig = reinterpret_cast<decltype(n.CommInitRankConfig)>(dlsym(h, "ncclCommInitRankConfig"));
    n.CommGetAsyncError = reinterpret_cast<decltype(n.CommGetAsyncError)>(dlsym(h, "ncclCommGetAsyncError"));
    n.CommAbort = reinterpret_cast<decltype(n.CommAbort)>(dlsym(h, "ncclCommAbort"));
    if (!n.GetUniqueId || !n.CommInitRank || !n.CommDestroy || !n.AllGather || !n.GetErrorString) {
        dlclose(h);
        return fvrt::fail(FV_ERR_NCCL, "libnccl.so.2 lacks a symbol this library needs");
    }
    n.lib = h;
    g_nccl = n;
    return FV_RAN;
}

#define FV_NCCL(expr)                                                                                  \
    do {                                                                                               \
        const int fv_nccl_rc = (expr);                                                                 \
        if (fv_nccl_rc != 0)                                                                           \
            return fvrt::fail(FV_ERR_NCCL, "%s: %s", #expr, fvsp::g_nccl.GetErrorString(fv_nccl_rc)); \
    } while (0)

struct Sp {
    int world = 1, rank = 0, seq = 0, bh = 0, groups = 1, bh_g = 0, dev = 0;
    int spare_sms = 24;
    double op_timeout_s = 120.0;  // how long settle() polls a call the non-blocking communicator left in progress
    int start = 0, len = 0, seg_rows = 0;
    std::vector<int> starts, lens;
    void* comm = nullptr;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ready = nullptr;
    cudaEvent_t arrived[kMaxGroups] = {};
    __nv_bfloat16* k_all[kMaxGroups] = {};  // [world, bh_g, seg_rows, 128] each
    __nv_bfloat16* v_all[kMaxGroups] = {};
    __nv_bfloat16* k_pad = nullptr;  // [bh, seg_rows, 128], only when this shard is shorter than the longest
    __nv_bfloat16* v_pad = nullptr;
    float* o1 = nullptr;    // [bh, len, 128]
    float* lse1 = nullptr;  // [bh, len]
};

// A communicator formed in non-blocking mode (the rendezvous with a deadline) answers ncclInProgress (7) from
// any call; the call has completed on the host side once ncclCommGetAsyncError stops saying so, and nothing
// else may be issued on the communicator before that.  Returns the settled NCCL result.
constexpr int kNcclInProgress = 7;
static int settle(Sp* s, int nrc) {
    if (nrc != kNcclInProgress || !g_nccl.CommGetAsyncError) return nrc;
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        int state = 0;
        const int q = g_nccl.CommGetAsyncError(s->comm, &state);
        if (q != 0) return q;
        if (state != kNcclInProgress) return state;
        timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        if ((double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec) > s->op_timeout_s) return kNcclInProgress;
        const timespec nap = {0, 20000};
        nanosleep(&nap, nullptr);
    }
}

static void release(Sp* s) {
    if (!s) return;
    if (s->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(s->comm);
    for (int g = 0; g < kMaxGroups; g++) {
        if (s->k_all[g]) cudaFree(s->k_all[g]);
        if (s->v_all[g]) cudaFree(s->v_all[g]);
        if (s->arrived[g]) cudaEventDestroy(s->arrived[g]);
    }
    if (s->k_pad) cudaFree(s->k_pad);
    if (s->v_pad) cudaFree(s->v_pad);
    if (s->o1) cudaFree(s->o1);
    if (s->lse1) cudaFree(s->lse1);
    if (s->ready) cudaEventDestroy(s->ready);
    if (s->comm_stream) cudaStreamDestroy(s->comm_stream);
    delete s;
}

// The other ranks whose shard holds a key some row of this shard may see (all of them without a mask); the
// block-causal predicate is crates/fastvideo-cudarc/src/rt/attn.rs:448-453.
static void visible_lens(int seq, int world, int rank, const int* starts, const int* lens, int mask_mode, int bt,
                         int window, int sink, int* lens_out) {
    for (int r = 0; r < world; r++) lens_out[r] = r == rank ? 0 : lens[r];
    if (mask_mode != FV_MASK_BLOCK_CAUSAL || lens[rank] == 0) return;
    if (bt < 1) bt = 1;
    const long long first = starts[rank], last = (long long)starts[rank] + lens[rank] - 1;
    long long hi = (last / bt + 1) * bt;
    if (hi > seq) hi = seq;
    long long lo = 0;
    if (window > 0) {
        lo = first / bt - window + 1;
        if (lo < 0) lo = 0;
        lo *= bt;
    }
    long long sink_hi = (long long)sink * bt;
    if (sink_hi > seq) sink_hi = seq;
    for (int r = 0; r < world; r++) {
        if (r == rank) continue;
        const long long s0 = starts[r], l = lens[r];
        const bool vis = l > 0 && ((s0 < hi && s0 + l > lo) || s0 < sink_hi);
        if (!vis) lens_out[r] = 0;
    }
}

static int forward(Sp* s, cudaStream_t stream, const void* q, const void* k, const void* v, void* out, int out_is_bf16,
                   float scale, int mask_mode, int bt, int window, int sink) {
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (dev != s->dev) return fvrt::fail(FV_ERR_INVALID, "sp: handle made on device %d, current device is %d", s->dev, dev);
    if (s->world == 1) {
        const int len = s->len, start = 0;
        return fv_sdpa_segments_bf16(stream, q, k, v, out, out_is_bf16, s->bh, s->len, 1, &len, &start, s->len, scale,
                                     mask_mode, bt, window, sink, 0, nullptr, nullptr, nullptr);
    }
    const size_t row_b = kD * sizeof(__nv_bfloat16);
    const void *ks = k, *vs = v;
    if (s->k_pad && s->len > 0) {  // rows past len stay zero from creation
        FV_CUDA(cudaMemcpy2DAsync(s->k_pad, s->seg_rows * row_b, k, s->len * row_b, s->len * row_b, s->bh,
                                  cudaMemcpyDeviceToDevice, stream));
        FV_CUDA(cudaMemcpy2DAsync(s->v_pad, s->seg_rows * row_b, v, s->len * row_b, s->len * row_b, s->bh,
                                  cudaMemcpyDeviceToDevice, stream));
    }
    if (s->k_pad) {
        ks = s->k_pad;
        vs = s->v_pad;
    }
    // The exchange starts once this rank's shard is final, and runs beside pass 1.
    FV_CUDA(cudaEventRecord(s->ready, stream));
    FV_CUDA(cudaStreamWaitEvent(s->comm_stream, s->ready, 0));
    const size_t group_elems = (size_t)s->bh_g * s->seg_rows * kD;
    for (int g = 0; g < s->groups; g++) {
        FV_NCCL(settle(s, g_nccl.AllGather(static_cast<const __nv_bfloat16*>(ks) + g * group_elems, s->k_all[g], group_elems, kNcclBf16,
                                           s->comm, s->comm_stream)));
        FV_NCCL(settle(s, g_nccl.AllGather(static_cast<const __nv_bfloat16*>(vs) + g * group_elems, s->v_all[g], group_elems, kNcclBf16,
                                           s->comm, s->comm_stream)));
        FV_CUDA(cudaEventRecord(s->arrived[g], s->comm_stream));
    }
    if (s->len == 0) {  // more ranks than tokens: this rank only takes part in the exchange
        for (int g = 0; g < s->groups; g++) FV_CUDA(cudaStreamWaitEvent(stream, s->arrived[g], 0));
        return FV_RAN;
    }
    std::vector<int> lens2(s->world);
    visible_lens(s->seq, s->world, s->rank, s->starts.data(), s->lens.data(), mask_mode, bt, window, sink, lens2.data());
    bool any = false;
    for (int r = 0; r < s->world; r++) any = any || lens2[r] > 0;
    // From here on the gathers are enqueued and read this rank's shard: whatever happens, the caller's stream
    // must not run ahead of them.
    auto wait_all = [&]() {
        for (int g = 0; g < s->groups; g++) cudaStreamWaitEvent(stream, s->arrived[g], 0);
    };
    const int len1 = s->len, start1 = s->start;
    // The gathers' copy kernels run beside pass 1: leave them SMs (FV_SP_SPARE_SMS, default 24), or the persistent
    // attention CTAs that find no SM start when the gathers end and finish that much later.
    if (s->world > 1) fv_hint_spare_sms(s->spare_sms);
    if (!any) {  // no row of this shard sees a key of another shard: pass 1 is the result
        rc = fv_sdpa_segments_bf16(stream, q, ks, vs, out, out_is_bf16, s->bh, s->len, 1, &len1, &start1, s->seg_rows, scale,
                                   mask_mode, bt, window, sink, s->start, nullptr, nullptr, nullptr);
    } else {
        rc = fv_sdpa_segments_bf16(stream, q, ks, vs, s->o1, 0, s->bh, s->len, 1, &len1, &start1, s->seg_rows, scale, mask_mode,
                                   bt, window, sink, s->start, s->lse1, nullptr, nullptr);
    }
    if (rc != FV_RAN) {
        wait_all();
        return rc;
    }
    const size_t q_group = (size_t)s->bh_g * s->len * kD;
    for (int g = 0; g < s->groups; g++) {
        // Also when pass 2 is skipped: the gather reads this rank's shard, which the caller may rewrite after this call.
        FV_CUDA(cudaStreamWaitEvent(stream, s->arrived[g], 0));
        if (!any) continue;
        void* og = out_is_bf16 ? static_cast<void*>(static_cast<__nv_bfloat16*>(out) + g * q_group)
                               : static_cast<void*>(static_cast<float*>(out) + g * q_group);
        rc = fv_sdpa_segments_bf16(stream, static_cast<const __nv_bfloat16*>(q) + g * q_group, s->k_all[g], s->v_all[g], og,
                                   out_is_bf16, s->bh_g, s->len, s->world, lens2.data(), s->starts.data(), s->seg_rows, scale,
                                   mask_mode, bt, window, sink, s->start, nullptr, s->o1 + g * q_group,
                                   s->lse1 + (size_t)g * s->bh_g * s->len);
        if (rc != FV_RAN) {
            wait_all();
            return rc;
        }
    }
    return FV_RAN;
}

// Rendezvous with a deadline.  ncclCommInitRank blocks for as long as a rank is missing; with NCCL's
// non-blocking mode the communicator is polled instead and, when the deadline passes, aborted: the caller
// gets FV_ERR_NCCL and a usable process back.  (Needs nccl.h at build time for ncclConfig_t and NCCL >= 2.14
// at run time; otherwise the blocking call is all there is.)
static int init_comm(Sp* s, const NcclId& id, int world, int rank, double timeout_s) {
#if FV_HAVE_NCCL_H
    if (timeout_s > 0 && g_nccl.CommInitRankConfig && g_nccl.CommGetAsyncError && g_nccl.CommAbort) {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.blocking = 0;
        int nrc = g_nccl.CommInitRankConfig(&s->comm, world, id, rank, &cfg);
        if (nrc != 0 && nrc != (int)ncclInProgress)
            return fvrt::fail(FV_ERR_NCCL, "ncclCommInitRankConfig: %s", g_nccl.GetErrorString(nrc));
        timespec t0;
        clock_gettime(CLOCK_MONOTONIC, &t0);
        for (;;) {
            int state = 0;
            nrc = g_nccl.CommGetAsyncError(s->comm, &state);
            if (nrc != 0) return fvrt::fail(FV_ERR_NCCL, "ncclCommGetAsyncError: %s", g_nccl.GetErrorString(nrc));
            if (state == 0) return FV_RAN;
            if (state != (int)ncclInProgress) {
                g_nccl.CommAbort(s->comm);
                s->comm = nullptr;
                return fvrt::fail(FV_ERR_NCCL, "sp: communicator of %d ranks failed to form: %s", world, g_nccl.GetErrorString(state));
            }
            timespec t1;
            clock_gettime(CLOCK_MONOTONIC, &t1);
            if ((double)(t1.tv_sec - t0.tv_sec) + 1e-9 * (double)(t1.tv_nsec - t0.tv_nsec) > timeout_s) {
                g_nccl.CommAbort(s->comm);
                s->comm = nullptr;
                return fvrt::fail(FV_ERR_NCCL, "sp: rank %d waited %.1f s for the other %d rank(s) of the communicator: rendezvous abandoned",
                                  rank, timeout_s, world - 1);
            }
            const timespec nap = {0, 2000000};
            nanosleep(&nap, nullptr);
        }
    }
#endif
    const int nrc = g_nccl.CommInitRank(&s->comm, world, id, rank);
    if (nrc != 0) return fvrt::fail(FV_ERR_NCCL, "ncclCommInitRank: %s", g_nccl.GetErrorString(nrc));
    return FV_RAN;
}

static int create(const void* unique_id, int world, int rank, int seq, int bh, int groups, double timeout_s, Sp** out) {
    if (!out) return fvrt::fail(FV_ERR_INVALID, "sp: null handle pointer");
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world) return fvrt::fail(FV_ERR_INVALID, "sp: rank %d out of world %d", rank, world);
    if (world > FV_MAX_SEGMENTS) return fvrt::fail(FV_ERR_INVALID, "sp: at most %d ranks", FV_MAX_SEGMENTS);
    if (seq < 1 || bh < 1) return fvrt::fail(FV_ERR_INVALID, "sp: seq and bh must be positive");
    if (world > 1 && !unique_id) return fvrt::fail(FV_ERR_INVALID, "sp: a communicator id is needed for more than one rank");
    int dev;
    int rc = fvrt::require_sm100(&dev);
    if (rc != FV_RAN) return rc;
    if (groups <= 0) groups = world >= 8 ? 2 : 1;
    if (groups > kMaxGroups || bh % groups != 0) groups = 1;
    Sp* s = new Sp();
    s->world = world;
    s->rank = rank;
    s->seq = seq;
    s->bh = bh;
    s->groups = groups;
    s->bh_g = bh / groups;
    s->dev = dev;
    s->starts.resize(world);
    s->lens.resize(world);
    fv_shard_ranges(seq, world, s->starts.data(), s->lens.data());
    s->start = s->starts[rank];
    s->len = s->lens[rank];
    for (int r = 0; r < world; r++) s->seg_rows = s->lens[r] > s->seg_rows ? s->lens[r] : s->seg_rows;
    if (world == 1) {
        *out = s;
        return FV_RAN;
    }
    auto bail = [&](int code) {
        release(s);
        return code;
    };
#define FV_TRY(expr)                                                                                     \
    do {                                                                                                 \
        const cudaError_t fv_e = (expr);                                                                 \
        if (fv_e != cudaSuccess) return bail(fvrt::fail(FV_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(fv_e))); \
    } while (0)
    rc = load_nccl();
    if (rc != FV_RAN) return bail(rc);
    int lo_prio = 0, hi_prio = 0;
    FV_TRY(cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio));
    // High priority: the attention kernel holds every SM with one large CTA, and NCCL's copy CTAs only run once all
    // of them are resident; at default priority they trickle in as attention CTAs retire.
    FV_TRY(cudaStreamCreateWithPriority(&s->comm_stream, cudaStreamNonBlocking, hi_prio));
    FV_TRY(cudaEventCreateWithFlags(&s->ready, cudaEventDisableTiming));
    const size_t group_bytes = (size_t)world * s->bh_g * s->seg_rows * kD * sizeof(__nv_bfloat16);
    for (int g = 0; g < groups; g++) {
        FV_TRY(cudaEventCreateWithFlags(&s->arrived[g], cudaEventDisableTiming));
        FV_TRY(cudaMalloc(&s->k_all[g], group_bytes));
        FV_TRY(cudaMalloc(&s->v_all[g], group_bytes));
        FV_TRY(cudaMemset(s->k_all[g], 0, group_bytes));
        FV_TRY(cudaMemset(s->v_all[g], 0, group_bytes));
    }
    if (s->len != s->seg_rows) {
        const size_t pad_bytes = (size_t)bh * s->seg_rows * kD * sizeof(__nv_bfloat16);
        FV_TRY(cudaMalloc(&s->k_pad, pad_bytes));
        FV_TRY(cudaMalloc(&s->v_pad, pad_bytes));
        FV_TRY(cudaMemset(s->k_pad, 0, pad_bytes));
        FV_TRY(cudaMemset(s->v_pad, 0, pad_bytes));
    }
    if (s->len > 0) {
        FV_TRY(cudaMalloc(&s->o1, (size_t)bh * s->len * kD * sizeof(float)));
        FV_TRY(cudaMalloc(&s->lse1, (size_t)bh * s->len * sizeof(float)));
    }
    FV_TRY(cudaDeviceSynchronize());
#undef FV_TRY
    NcclId id;
    memcpy(id.bytes, unique_id, sizeof(id.bytes));
    rc = init_comm(s, id, world, rank, timeout_s);
    if (rc != FV_RAN) return bail(rc);
    if (timeout_s > 0) s->op_timeout_s = timeout_s;
    if (const char* e = getenv("FV_SP_SPARE_SMS")) {
        const int n = atoi(e);
        if (n >= 0 && n <= 128) s->spare_sms = n;
    }
    // Every rank must describe the same problem: a rank with another seq, bh or group count would size its
    // gathers differently and the first exchange would never complete.  One small all-gather settles it here,
    // where a mismatch is an error return on every rank instead of a hang later.
    {
        int* shape_dev = nullptr;
        const int mine[4] = {seq, bh, groups, world};
        std::vector<int> all(4 * (size_t)world);
        cudaError_t e = cudaMalloc(&shape_dev, sizeof(int) * 4 * ((size_t)world + 1));
        if (e == cudaSuccess) e = cudaMemcpy(shape_dev + 4 * (size_t)world, mine, sizeof(mine), cudaMemcpyHostToDevice);
        int nrc = 0;
        if (e == cudaSuccess) nrc = settle(s, g_nccl.AllGather(shape_dev + 4 * (size_t)world, shape_dev, 16, /* ncclInt8 */ 0, s->comm, s->comm_stream));
        if (e == cudaSuccess && nrc == 0) e = cudaStreamSynchronize(s->comm_stream);
        if (e == cudaSuccess && nrc == 0) e = cudaMemcpy(all.data(), shape_dev, sizeof(int) * 4 * (size_t)world, cudaMemcpyDeviceToHost);
        if (shape_dev) cudaFree(shape_dev);
        if (nrc != 0) return bail(fvrt::fail(FV_ERR_NCCL, "sp: shape handshake: %s", g_nccl.GetErrorString(nrc)));
        if (e != cudaSuccess) return bail(fvrt::fail(FV_ERR_CUDA, "sp: shape handshake: %s", cudaGetErrorString(e)));
        for (int r = 0; r < world; r++)
            if (memcmp(&all[4 * (size_t)r], mine, sizeof(mine)) != 0)
                return bail(fvrt::fail(FV_ERR_INVALID, "sp: rank %d was created with seq %d, bh %d, groups %d, world %d; this rank (%d) with %d, %d, %d, %d",
                                       r, all[4 * r], all[4 * r + 1], all[4 * r + 2], all[4 * r + 3], rank, seq, bh, groups, world));
    }
    *out = s;
    return FV_RAN;
}

}  // namespace fvsp

extern "C" int fv_sp_unique_id(void* id_out) {
    fvrt::clear_error();
    if (!id_out) return fvrt::fail(FV_ERR_INVALID, "sp: null id buffer");
    int rc = fvsp::load_nccl();
    if (rc != FV_RAN) return rc;
    fvsp::NcclId id;
    FV_NCCL(fvsp::g_nccl.GetUniqueId(&id));
    memcpy(id_out, id.bytes, sizeof(id.bytes));
    return FV_RAN;
}

extern "C" int fv_sp_second_pass_lens(int seq, int world, int rank, int mask_mode, int block_tokens, int window, int sink,
                                      int* lens_out) {
    fvrt::clear_error();
    if (world < 1 || world > FV_MAX_SEGMENTS || rank < 0 || rank >= world || seq < 1 || !lens_out)
        return fvrt::fail(FV_ERR_INVALID, "sp: rank %d of %d ranks, %d tokens", rank, world, seq);
    int starts[FV_MAX_SEGMENTS], lens[FV_MAX_SEGMENTS];
    fv_shard_ranges(seq, world, starts, lens);
    fvsp::visible_lens(seq, world, rank, starts, lens, mask_mode, block_tokens, window, sink, lens_out);
    return FV_RAN;
}

extern "C" int fv_sp_create_timeout(const void* unique_id, int world, int rank, int seq, int bh, int groups,
                                    double timeout_seconds, void** sp_out) {
    fvrt::clear_error();
    fvsp::Sp* s = nullptr;
    const int rc = fvsp::create(unique_id, world, rank, seq, bh, groups, timeout_seconds, &s);
    if (sp_out) *sp_out = s;
    else if (s) fvsp::release(s);
    return rc;
}

extern "C" int fv_sp_create(const void* unique_id, int world, int rank, int seq, int bh, int groups, void** sp_out) {
    // FV_SP_INIT_TIMEOUT_S: seconds to wait for the other ranks (default 120; 0 = NCCL's own blocking rendezvous)
    const char* e = getenv("FV_SP_INIT_TIMEOUT_S");
    const double t = e ? atof(e) : 120.0;
    return fv_sp_create_timeout(unique_id, world, rank, seq, bh, groups, t, sp_out);
}

extern "C" int fv_sp_destroy(void* sp) {
    fvrt::clear_error();
    fvsp::release(static_cast<fvsp::Sp*>(sp));
    return FV_RAN;
}

extern "C" int fv_sp_info(void* sp, int* start, int* len, int* seg_rows, int* groups) {
    fvrt::clear_error();
    if (!sp) return fvrt::fail(FV_ERR_INVALID, "sp: null handle");
    const fvsp::Sp* s = static_cast<const fvsp::Sp*>(sp);
    if (start) *start = s->start;
    if (len) *len = s->len;
    if (seg_rows) *seg_rows = s->seg_rows;
    if (groups) *groups = s->groups;
    return FV_RAN;
}

extern "C" int fv_sp_forward_bf16(void* sp, void* stream, const void* q, const void* k, const void* v, void* out,
                                  int out_is_bf16, float scale, int mask_mode, int block_tokens, int window, int sink) {
    fvrt::clear_error();
    if (!sp) return fvrt::fail(FV_ERR_INVALID, "sp: null handle");
    if ((!q || !k || !v || !out) && static_cast<fvsp::Sp*>(sp)->len > 0) return fvrt::fail(FV_ERR_INVALID, "sp: null operand");
    return fvsp::forward(static_cast<fvsp::Sp*>(sp), (cudaStream_t)stream, q, k, v, out, out_is_bf16, scale, mask_mode,
                         block_tokens, window, sink);
}

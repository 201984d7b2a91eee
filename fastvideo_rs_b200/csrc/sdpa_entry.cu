// C face of the chooser (sdpa_rule.cpp) and the one attention entry, fv_sdpa, which mirrors
// rt::sdpa::sdpa (crates/fastvideo-cudarc/src/rt/sdpa.rs:141-164): validate BHSD, let the rule
// choose, run the step when it is this library's kernel, decline otherwise.
#include "fv_runtime.h"
#include "sdpa_rule.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#include <algorithm>
#include <string>

using namespace fvrule;

static Probe to_probe(const fv_probe* c) {
    Probe p;
    p.backend = (Backend)c->backend;
    p.sp_world = (size_t)std::max(c->sp_world, 1);
    p.mma_default = c->mma_default != 0;
    p.has_sage = c->has_sage != 0;
    p.sage_min_seq = (size_t)std::max(c->sage_min_seq, 0);
    p.fp8_dense = c->fp8_dense != 0;
    p.causal_flash = c->causal_flash != 0;
    p.kernel_choice = std::string(c->kernel_choice, strnlen(c->kernel_choice, sizeof(c->kernel_choice)));
    p.has_sm = c->has_sm != 0;
    p.sm_major = c->sm_major;
    p.sms = (size_t)std::max(c->sms, 1);
    p.dc_loaded = c->dc_loaded != 0;
    p.b200_loaded = c->b200_loaded != 0;
    p.auto_mode = c->auto_timed ? AutoMode::Timed : AutoMode::Rule;
    p.cudnn_has_plan = c->cudnn_has_plan != 0;
    return p;
}

static std::string env_lower(const char* name, const char* dflt) {
    const char* v = getenv(name);
    std::string s = v ? v : dflt;
    for (auto& ch : s) ch = (char)tolower((unsigned char)ch);
    return s;
}
static bool env_bool(const char* name, bool dflt) {
    const char* v = getenv(name);
    if (!v || !*v) return dflt;
    std::string s = v;
    for (auto& ch : s) ch = (char)tolower((unsigned char)ch);
    if (s == "0" || s == "false" || s == "off" || s == "no") return false;
    if (s == "1" || s == "true" || s == "on" || s == "yes") return true;
    return dflt;
}

extern "C" void fv_probe_default(fv_probe* o) {
    memset(o, 0, sizeof(*o));
    o->backend = FV_BACKEND_DENSE;
    o->sp_world = 1;
    o->mma_default = 1;
    o->causal_flash = 1;
    strcpy(o->kernel_choice, "auto");
    o->has_sm = 1;
    o->sm_major = 10;
    o->sms = 148;
    o->b200_loaded = 1;
}

extern "C" void fv_probe_live(fv_probe* o) {
    fv_probe_default(o);
    o->backend = (int)parse_backend(env_lower("FASTVIDEO_SDPA", "dense"));
    const char* w = getenv("FASTVIDEO_SP_WORLD");
    o->sp_world = std::max(w ? atoi(w) : 1, 1);
    o->causal_flash = env_bool("FASTVIDEO_WAN_CAUSAL_FLASH", true) ? 1 : 0;
    const std::string kc = env_lower("FASTVIDEO_FLASH_KERNEL", "auto");
    strncpy(o->kernel_choice, kc.c_str(), sizeof(o->kernel_choice) - 1);
    o->kernel_choice[sizeof(o->kernel_choice) - 1] = 0;
    o->auto_timed = parse_auto_mode(env_lower("FASTVIDEO_SDPA_AUTO", "rule")) == AutoMode::Timed;
    int dev = -1, major = 0, sms = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 &&
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess) {
        o->has_sm = 1;
        o->sm_major = major;
        o->sms = std::max(sms, 1);
        o->mma_default = major >= 8;
        o->b200_loaded = major == 10;
    } else {
        cudaGetLastError();
        o->has_sm = 0;
        o->sm_major = 0;
        o->sms = 1;
        o->mma_default = 0;
        o->b200_loaded = 0;
    }
}

extern "C" int fv_rule_parse_backend(const char* v) { return (int)parse_backend(v ? v : ""); }
extern "C" int fv_rule_parse_auto_timed(const char* v) { return parse_auto_mode(v ? v : "") == AutoMode::Timed; }
extern "C" int fv_rule_parse_kernel_override(const char* v) {
    FlashKernel k;
    return parse_kernel_override(v ? v : "", &k) ? (int)k : -1;
}
extern "C" int fv_rule_flash_v2_fills(size_t sq, size_t bh, size_t sms) { return flash_v2_fills(sq, bh, sms); }
extern "C" int fv_rule_pick(int sm_major, size_t sq, size_t sk, size_t d) { return (int)pick(sm_major, sq, sk, d); }
extern "C" void fv_rule_shape_of(const size_t q[4], const size_t k[4], const size_t v[4], size_t* sq, size_t* sk,
                                 int* dims_ok) {
    const Shape s = Shape::of(q, k, v);
    if (sq) *sq = s.sq;
    if (sk) *sk = s.sk;
    if (dims_ok) *dims_ok = s.has_dims;
}
extern "C" int fv_rule_dense_route(const size_t q[4], const size_t k[4], const size_t v[4], int masked, int out_bf16,
                                   const fv_probe* p, fv_step steps[8]) {
    const auto r = dense_route(Shape::of(q, k, v), masked != 0, out_bf16 != 0, to_probe(p));
    for (size_t i = 0; i < r.size() && i < 8; i++) steps[i] = fv_step{(int)r[i].kind, r[i].out_bf16, (int)r[i].retired};
    return (int)r.size();
}
extern "C" int fv_rule_flash_kernel_for(size_t sq, size_t bh, size_t sms, const fv_probe* p) {
    return (int)flash_kernel_for(sq, bh, sms, to_probe(p));
}
extern "C" int fv_rule_mma_kernel(const size_t q[4], const size_t k[4], const size_t v[4], int out_bf16,
                                  const fv_probe* p, int* kernel, int* sm_major) {
    const MmaKernel m = mma_kernel(Shape::of(q, k, v), out_bf16 != 0, to_probe(p));
    if (kernel) *kernel = (int)m.kernel;
    if (sm_major) *sm_major = m.sm_major;
    return (int)m.kind;
}
extern "C" int fv_rule_fp8_first(const fv_probe* p) { return fp8_first(to_probe(p)); }
extern "C" int fv_rule_block_causal_first(const fv_probe* p) { return block_causal_first(to_probe(p)); }
extern "C" int fv_rule_vdn_window_first(const fv_probe* p) { return vdn_window_first(to_probe(p)); }
extern "C" int fv_rule_kv_window_flash(int flash, const fv_probe* p) { return kv_window_flash(flash, to_probe(p)); }
extern "C" int fv_rule_mma_sdpa_supported(size_t b, size_t h, size_t sq, size_t sk, size_t d, int sm_major) {
    return mma_sdpa_supported(b, h, sq, sk, d, sm_major);
}

extern "C" void fv_shard_ranges(int seq, int world, int* start, int* len) {
    if (world < 1) world = 1;
    const int base = seq / world, rem = seq % world;
    int s = 0;
    for (int r = 0; r < world; r++) {
        len[r] = base + (r < rem ? 1 : 0);
        start[r] = s;
        s += len[r];
    }
}

// The Mma step: this library's kernel when the rule picks it, else not ours.
// With a workspace, an unmasked call whose grid fills the SMs a ragged number of times is cut along the keys.
static int run_mma(void* stream, const void* q, const void* k, const void* v, const Shape& sh, bool out_bf16,
                   const Probe& p, float scale, void* out, int mask_mode, int bt, int win, int sink,
                   void* ws = nullptr, size_t ws_bytes = 0) {
    const MmaKernel m = mma_kernel(sh, out_bf16, p);
    if (m.kind != MmaKind::Fixed || m.kernel != FlashKernel::B200) return FV_DECLINED;
    if (!sh.has_dims) return FV_DECLINED;
    const Dims& d = sh.dims;
    if (!mma_sdpa_supported(d.b, d.h, d.sq, d.sk, d.d, p.has_sm ? p.sm_major : 0)) return FV_DECLINED;
    if (ws && mask_mode == FV_MASK_NONE && d.d == 128 && d.sq <= 0x3fffffff && d.sk <= 0x3fffffff) {
        const int splits = fv_sdpa_splitkv_choose((int)(d.b * d.h), (int)d.sq, (int)d.sk, (int)p.sms);
        if (splits > 1 && fv_sdpa_splitkv_workspace_bytes((int)(d.b * d.h), (int)d.sq, splits) <= ws_bytes)
            return fv_sdpa_splitkv_bf16(stream, q, k, v, out, out_bf16 ? 1 : 0, (int)(d.b * d.h), (int)d.sq, (int)d.sk,
                                        (int)d.d, scale, splits, 0, ws, ws_bytes);
    }
    return fv_sdpa_dense_bf16(stream, q, k, v, out, out_bf16 ? 1 : 0, (int)(d.b * d.h), (int)d.sq, (int)d.sk, (int)d.d,
                              scale, mask_mode, bt, win, sink, 0);
}

extern "C" int fv_sdpa(void* stream, const void* q, const void* k, const void* v, const size_t q_shape[4],
                       const size_t k_shape[4], const size_t v_shape[4], const fv_plan* plan, const fv_probe* probe,
                       void* out, int out_is_bf16) {
    return fv_sdpa_ws(stream, q, k, v, q_shape, k_shape, v_shape, plan, probe, out, out_is_bf16, nullptr, 0);
}

extern "C" size_t fv_sdpa_ws_bytes(const size_t q_shape[4], const size_t k_shape[4], const fv_plan* plan,
                                   const fv_probe* probe) {
    if (!q_shape || !k_shape || !plan) return 0;
    if (plan->kind != FV_PLAN_KV_WINDOW && !(plan->kind == FV_PLAN_DENSE && !plan->has_mask)) return 0;
    fv_probe live;
    if (!probe) {
        fv_probe_live(&live);
        probe = &live;
    }
    const size_t bh = q_shape[0] * q_shape[1];
    if (q_shape[3] != 128 || bh == 0 || bh > 65535 || q_shape[2] > 0x3fffffff || k_shape[2] > 0x3fffffff) return 0;
    const int splits = fv_sdpa_splitkv_choose((int)bh, (int)q_shape[2], (int)k_shape[2], probe->sms);
    return splits > 1 ? fv_sdpa_splitkv_workspace_bytes((int)bh, (int)q_shape[2], splits) : 0;
}

extern "C" int fv_sdpa_ws(void* stream, const void* q, const void* k, const void* v, const size_t q_shape[4],
                          const size_t k_shape[4], const size_t v_shape[4], const fv_plan* plan, const fv_probe* probe,
                          void* out, int out_is_bf16, void* workspace, size_t workspace_bytes) {
    fvrt::clear_error();
    if (!q_shape || !k_shape || !v_shape || !plan) return fvrt::fail(FV_ERR_INVALID, "sdpa expects BHSD");
    fv_probe live;
    if (!probe) {
        fv_probe_live(&live);
        probe = &live;
    }
    const Probe p = to_probe(probe);
    const Shape sh = Shape::of(q_shape, k_shape, v_shape);
    const float d = (float)q_shape[3];
    const float scale = plan->has_scale ? plan->scale : 1.0f / sqrtf(d);
    switch (plan->kind) {
        case FV_PLAN_DENSE: {
            // fp8_first is a kernel of the reference's own; if it is on, that step comes first and is not ours.
            if (plan->fp8_first && fp8_first(p)) return FV_DECLINED;
            const auto route = dense_route(sh, plan->has_mask != 0, out_is_bf16 != 0, p);
            for (const Step& st : route) {
                if (st.kind == StepKind::Retired)
                    return fvrt::fail(FV_ERR_INVALID, "FASTVIDEO_SDPA=%s is retired: unset FASTVIDEO_SDPA for dense attention",
                                      st.retired == Backend::Sparse ? "sparse" : "host");
                if (st.kind != StepKind::Mma) return FV_DECLINED;  // an earlier step of the route is the caller's
                const int rc = run_mma(stream, q, k, v, sh, st.out_bf16 != 0, p, scale, out, FV_MASK_NONE, 0, 0, 0,
                                       plan->has_mask ? nullptr : workspace, workspace_bytes);
                return rc;  // ran, declined (caller continues with the next step), or error
            }
            return FV_DECLINED;
        }
        case FV_PLAN_BLOCK_CAUSAL: {
            if (!block_causal_first(p)) return FV_DECLINED;  // dense additive mask: the composed step
            if (plan->block_tokens < 1 || plan->window < 0 || plan->sink < 0)
                return fvrt::fail(FV_ERR_INVALID, "block_causal: block_tokens >= 1, window >= 0, sink >= 0");
            // device_mma_sdpa_causal runs where the fused kernel runs; ours when the seam says so.
            Probe pc = p;
            const FlashKernel fk = flash_kernel_for(sh.sq, sh.has_dims ? sh.dims.b * sh.dims.h : 1, p.sms, pc);
            if (fk != FlashKernel::B200) return FV_DECLINED;
            if (!sh.has_dims) return FV_DECLINED;
            const Dims& dd = sh.dims;
            if (!mma_sdpa_supported(dd.b, dd.h, dd.sq, dd.sk, dd.d, p.has_sm ? p.sm_major : 0)) return FV_DECLINED;
            return fv_sdpa_dense_bf16(stream, q, k, v, out, out_is_bf16, (int)(dd.b * dd.h), (int)dd.sq, (int)dd.sk,
                                      (int)dd.d, scale, FV_MASK_BLOCK_CAUSAL, plan->block_tokens, plan->window,
                                      plan->sink, 0);
        }
        case FV_PLAN_KV_WINDOW: {
            if (!kv_window_flash(plan->kv_flash, p)) return FV_DECLINED;  // the f32 composed reference
            const auto route = dense_route(sh, false, out_is_bf16 != 0, p);
            for (const Step& st : route) {
                if (st.kind == StepKind::Retired) return fvrt::fail(FV_ERR_INVALID, "FASTVIDEO_SDPA backend is retired");
                if (st.kind != StepKind::Mma) return FV_DECLINED;
                return run_mma(stream, q, k, v, sh, st.out_bf16 != 0, p, 1.0f / sqrtf(d), out, FV_MASK_NONE, 0, 0, 0,
                               workspace, workspace_bytes);
            }
            return FV_DECLINED;
        }
        case FV_PLAN_COMPOSED:
        case FV_PLAN_VDN_WINDOW:
            return FV_DECLINED;
        default:
            return fvrt::fail(FV_ERR_INVALID, "sdpa: unknown plan kind %d", plan->kind);
    }
}

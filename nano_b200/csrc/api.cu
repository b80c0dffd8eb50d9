// api.cu -- the entry points of include/nano_b200.h that every model family shares, and the registry that picks the family.
//
//   nb200_engine_create      a model-file IMAGE: the BD4SURLM magic selects the Nano family (engine.cu)
//   nb200_engine_create_dir  a model FOLDER (config.json + model.safetensors): config "architecture" selects the family by name
// Everything else here forwards through the engine's EngineOps table (family.h).
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <string>

#include "family.h"
#include "modeldir.h"

namespace nb {
namespace { thread_local std::string g_err; }

int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}
}  // namespace nb

using nb::fail;

namespace {
inline nb::EngineBase *base(nb200_engine *e) { return reinterpret_cast<nb::EngineBase *>(e); }
inline const nb::EngineBase *base(const nb200_engine *e) { return reinterpret_cast<const nb::EngineBase *>(e); }

// config.json "architecture" -> family.  A design that is a list of typed layers (mixers + feed-forwards) is served by the
// layered runtime; more names join it by registering their layer types there.
typedef int (*DirCreate)(nb200_engine **, const nb::ModelDir *, uint32_t, int, uint32_t);
struct DirFamily { const char *architecture; DirCreate create; const char *unit; };
const DirFamily kDirFamilies[] = {
    {"Famudra", nb_family_layered_create, "layered.cu"},
    {"Rakarax", nb_family_layered_create, "layered.cu"},
    {"Gokinex", nb_family_layered_create, "layered.cu"},
    {"Vumunex", nb_family_layered_create, "layered.cu"},
};
}  // namespace

#define NB_OP(e, op) \
    if (!(e)) return fail(NB200_EINVAL, "null engine"); \
    if (!base(e)->ops->op) return fail(NB200_EINVAL, #op " is not available for this model family")

extern "C" {

const char *nb200_last_error(void) { return nb::g_err.c_str(); }

int nb200_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

int nb200_engine_create(nb200_engine **out, const uint8_t *image, uint64_t image_bytes, uint32_t max_seq_len, int device, uint32_t flags) {
    if (!out || !image || image_bytes < 8) return fail(NB200_EINVAL, "bad arguments");
    if (!nb_family_nano_create) return fail(NB200_EINVAL, "the model-file family (engine.cu) is not part of this build of the library");
    return nb_family_nano_create(out, image, image_bytes, max_seq_len, device, flags);
}

int nb200_engine_create_dir(nb200_engine **out, const char *model_dir, uint32_t max_tokens, int device, uint32_t flags) {
    if (!out || !model_dir || max_tokens == 0) return fail(NB200_EINVAL, "bad arguments");
    *out = nullptr;
    nb::ModelDir dir;
    std::string err;
    if (nb::modeldir_open(model_dir, &dir, &err)) return fail(NB200_EINVAL, "%s", err.c_str());
    const nb::Json *arch = dir.config.get("architecture");
    if (!arch || arch->t != nb::Json::Str) return fail(NB200_EINVAL, "config.json names no \"architecture\"");
    for (const DirFamily &f : kDirFamilies) {
        if (arch->str != f.architecture) continue;
        if (!f.create) return fail(NB200_EINVAL, "architecture %s needs %s, which is not part of this build of the library", f.architecture, f.unit);
        if (nb200_device_count() <= 0) return fail(NB200_ENODEV, "no CUDA device: nano_b200 has no CPU path");
        return f.create(out, &dir, max_tokens, device, flags);
    }
    return fail(NB200_EINVAL, "unknown architecture \"%s\"", arch->str.c_str());
}

void nb200_engine_destroy(nb200_engine *e) { if (e) base(e)->ops->destroy(e); }

int nb200_get_config(const nb200_engine *e, nb200_config *cfg) {
    if (!e || !cfg) return fail(NB200_EINVAL, "null argument");
    return base(e)->ops->get_config(e, cfg);
}
int nb200_forward(nb200_engine *e, uint32_t token, uint32_t pos, uint32_t is_causal) { NB_OP(e, forward); return base(e)->ops->forward(e, token, pos, is_causal); }
int nb200_read_logits(nb200_engine *e, float *host_logits) { NB_OP(e, read_logits); return base(e)->ops->read_logits(e, host_logits); }
int nb200_next_greedy(nb200_engine *e, const uint32_t *ids, uint32_t pos, int is_prefilling, float penalty, uint32_t *next) {
    NB_OP(e, next_greedy); return base(e)->ops->next_greedy(e, ids, pos, is_prefilling, penalty, next);
}
int nb200_next_sampled(nb200_engine *e, const uint32_t *ids, uint32_t pos, float penalty, float temperature, float top_p, float coin,
                       uint32_t *next, uint32_t *top6) {
    NB_OP(e, next_sampled); return base(e)->ops->next_sampled(e, ids, pos, penalty, temperature, top_p, coin, next, top6);
}
int nb200_decode_greedy(nb200_engine *e, uint32_t *ids, uint32_t n_prompt, uint32_t n_total, float penalty, float *prefill_ms, float *device_ms) {
    NB_OP(e, decode_greedy); return base(e)->ops->decode_greedy(e, ids, n_prompt, n_total, penalty, prefill_ms, device_ms);
}
int nb200_seq_open(nb200_engine *e, uint32_t *seq) { NB_OP(e, seq_open); return base(e)->ops->seq_open(e, seq); }
int nb200_seq_close(nb200_engine *e, uint32_t seq) { NB_OP(e, seq_close); return base(e)->ops->seq_close(e, seq); }
int nb200_step(nb200_engine *e, uint32_t seq, const uint32_t *tokens, uint32_t n, const uint32_t *want, uint32_t n_want, float *logits) {
    NB_OP(e, step); return base(e)->ops->step(e, seq, tokens, n, want, n_want, logits);
}
int nb200_step_timed(nb200_engine *e, uint32_t seq, const uint32_t *tokens, uint32_t n, uint32_t reps, float *ms) {
    NB_OP(e, step_timed); return base(e)->ops->step_timed(e, seq, tokens, n, reps, ms);
}
int nb200_read_residual(nb200_engine *e, uint32_t run, float *dst, uint32_t count) { NB_OP(e, read_residual); return base(e)->ops->read_residual(e, run, dst, count); }

uint64_t nb200_kernel_launches(const nb200_engine *e) { return e ? base(e)->launches : 0; }
uint32_t nb200_launches_per_token(const nb200_engine *e) { return e ? base(e)->launches_per_token : 0; }
uint64_t nb200_weight_bytes(const nb200_engine *e) { return e ? base(e)->weight_bytes : 0; }

}  // extern "C"

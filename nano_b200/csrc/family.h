// family.h -- the model-family registry of libnano_b200.so.
//
// An engine handle (nb200_engine *) points at an object whose first base is nb::EngineBase: a table of the entry points every
// family implements (step, generation, logits) plus the counters the C-ABI reports.  api.cu owns the public symbols shared by all
// families and dispatches through that table; each family lives in translation units of its own and is reached through ONE weak
// creation symbol, so a library linked without a family still loads and answers "not part of this build" for its models:
//     nb_family_nano_create     engine.cu    BD4SURLM model-file images (Nano / Qwen2 / Qwen3 decoders, F32 / Q80 / Q4K)
//     nb_family_layered_create  layered.cu   config.json + model.safetensors folders whose config lists its layers (Famudra, Rakarax, Gokinex)
#pragma once
#include <stdint.h>

#include "../../include/nano_b200.h"

namespace nb {

// records the message nb200_last_error() returns (per thread) and hands `code` back
int fail(int code, const char *fmt, ...);

#define NB_CK(call)                                                                                                       \
    do {                                                                                                                  \
        cudaError_t e_ = (call);                                                                                          \
        if (e_ != cudaSuccess)                                                                                            \
            return ::nb::fail(NB200_ECUDA, "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
    } while (0)

struct EngineOps {
    void (*destroy)(nb200_engine *);
    int (*get_config)(const nb200_engine *, nb200_config *);
    int (*forward)(nb200_engine *, uint32_t token, uint32_t pos, uint32_t is_causal);
    int (*read_logits)(nb200_engine *, float *);
    int (*next_greedy)(nb200_engine *, const uint32_t *ids, uint32_t pos, int is_prefilling, float penalty, uint32_t *next);
    int (*next_sampled)(nb200_engine *, const uint32_t *ids, uint32_t pos, float penalty, float temperature, float top_p, float coin,
                        uint32_t *next, uint32_t *top6);
    int (*decode_greedy)(nb200_engine *, uint32_t *ids, uint32_t n_prompt, uint32_t n_total, float penalty, float *prefill_ms, float *device_ms);
    // sequence interface (families with a state manager for several live requests); null where a family has one implicit sequence
    int (*seq_open)(nb200_engine *, uint32_t *seq);
    int (*seq_close)(nb200_engine *, uint32_t seq);
    int (*step)(nb200_engine *, uint32_t seq, const uint32_t *tokens, uint32_t n, const uint32_t *want, uint32_t n_want, float *logits);
    int (*read_residual)(nb200_engine *, uint32_t run, float *dst, uint32_t count);
    int (*step_timed)(nb200_engine *, uint32_t seq, const uint32_t *tokens, uint32_t n, uint32_t reps, float *ms);
};

struct EngineBase {
    const EngineOps *ops = nullptr;
    uint64_t launches = 0, weight_bytes = 0;
    uint32_t launches_per_token = 0;
};

// a model folder as the registry hands it to a family: the parsed config and the tensor directory of model.safetensors
struct ModelDir;

}  // namespace nb

extern "C" {
int nb_family_nano_create(nb200_engine **out, const uint8_t *image, uint64_t image_bytes, uint32_t max_seq_len, int device,
                          uint32_t flags) __attribute__((weak));
int nb_family_layered_create(nb200_engine **out, const nb::ModelDir *dir, uint32_t max_tokens, int device, uint32_t flags)
    __attribute__((weak));
}

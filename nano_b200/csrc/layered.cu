// layered.cu -- the layered model family of libnano_b200.so: decoders described by config.json as a list of typed layers
// (a token mixer + an optional feed-forward each, over an fp32 residual stream), loaded from model.safetensors.
//
// Registered designs (config.json "architecture"):
// "Rakarax" -- sequential sublayers with a norm before and after each one, x <- x + norm1b(mixer(norm1 x)), then
// x <- x + norm2b(ff(norm2 x)), vector-gain RMS norms stored around zero, a learned position row added to the embedding; mixers
// "retention" (rotary linear attention with a fixed decay per head, fp32 state) and "parallel" (a sliding-window grouped-query
// attention whose scores are mixed across heads, side by side with a Mamba selective scan, summed with fixed scales); feed-forward
// "dense" (PolyNorm activation); a layer may use another layer's weights ("weights_of") with cache and state of its own.
// "Gokinex" -- the same sequential form with Dynamic-Tanh norms (tanh(alpha u) w + b); the token row times a fixed scale plus a
// hashed row for the (previous, current) token pair; mixers "attention" (grouped-query differential attention: two softmax maps per
// head over the same values, rotary positions on interleaved pairs with frequencies rescaled by wavelength, optionally on another
// layer's keys and values) and "mamba2" (state-space duality with a scalar decay per head and token); feed-forward "dense" (gated
// gelu) or "moe" (silu experts chosen by sigmoid scores that weight the expert's input, plus a shared expert behind a sigmoid gate).
// "Vumunex" -- pre-norm sequential sublayers over `streams` copies of the residual (hyper-connections: a sublayer reads a weighted sum
// of the streams through a bias-free layer norm and its output, times a per-channel layer scale and one multiplier for the whole model,
// returns into every stream while a small matrix mixes the streams); the token row times a fixed scale; mixers "latent_attention"
// (direct queries against an RMS-normed key/value latent, no positions, a sliding window, a softmax with one learned extra term per
// head in its denominator, a sigmoid output gate) and "latent_attention_2" (the same latent with a rotated key part shared by the heads
// beside it, rotary positions on interleaved pairs, causal, ordinary softmax, output gate); feed-forward "dense" (exact gelu) or "moe"
// (clamped gated experts chosen by their softmax scores, weighted on the way out, plus a shared expert); "loop" as below, without
// the embedding added again.
// "Famudra" -- parallel layers  x <- x + (mixer(shift(norm1 x)) + ff(norm2 x))  with scalar-gain RMS norms and a
// token shift on the mixer input; mixers "rglru" (gelu branch x conv + real-gated linear recurrent unit) and "latent_attention"
// (queries and keys/values through normed low-rank latents, no positions, causal softmax); feed-forward "moe" (top-k routed
// squared-relu experts + a shared expert); a span of layers may run several times with the same weights ("loop"), each pass with
// cache and state of its own and the embedding output added again before every pass but the first.
//
// Host side of the family:
//   loader         config -> layer table; tensors -> HBM in the compute type (bf16 as stored, or widened to fp32 with NB200_FLAG_F32),
//                  fused where one product serves two projections ([y | x] of the recurrent block, [query latent | kv latent],
//                  [recurrence gate | input gate] blocks, experts stacked), W_uk transposed per head so queries can be absorbed
//   state manager  sequences = {cache pages, one state slot}.  Pages of kPage tokens come from a LIFO free list and hold the rows
//                  of EVERY attention layer run (latents, or key/value rows of a window attention); a slot holds, per layer run,
//                  what the run carries from token to token: the previous mixer input (token shift), fp32 recurrent states
//                  (rglru, retention, selective scan) and convolution tails.  Slots are zeroed when a sequence opens.
//   step           a portion of n tokens is cut into chunks of <= chunk_cap tokens; each chunk runs every layer run with the prefill
//                  kernels (n > kGemvMaxM) or the decode kernels; logits only where asked
//   generation     the C-ABI's forward / next_greedy / next_sampled / decode_greedy on one implicit sequence; the greedy loop feeds
//                  the chosen token back on the device
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <string>
#include <vector>

#include "family.h"
#include "layered_kernels.cuh"
#include "layered_mixers.cuh"
#include "layered_mixers2.cuh"
#include "layered_mixers3.cuh"
#include "modeldir.h"
#include "sample_host.h"

using nb::fail;
using namespace nb::lm;

#define CK(call) NB_CK(call)

namespace {

struct Weight { void *p = nullptr; uint32_t rows = 0, cols = 0; };

enum MixerType { MIX_RGLRU = 0, MIX_LATENT_ATTN = 1, MIX_RETENTION = 2, MIX_WINDOW_SSM = 3, MIX_DIFF_ATTN = 4, MIX_SSD = 5 };
// how a layer combines its sublayers: Famudra's parallel form with a token shift and scalar-gain norms, or sequential sublayers
// between an input norm and an output norm each (vector gains stored around zero)
// or pre-norm sublayers over hyper-connected residual streams (bias-free layer norms)
enum LayerForm { FORM_PARALLEL_SHIFT = 0, FORM_SANDWICH = 1, FORM_HYPER = 2 };
enum FfKind { FF_NONE = 0, FF_MOE = 1, FF_DENSE_POLY = 2, FF_DENSE_GLU = 3, FF_MOE_SCORED = 4, FF_DENSE_GELU = 5 };
// the norms of the sequential form: unit RMS times a vector gain stored around zero, or Dynamic Tanh
enum NormKind { NORM_RMS_ZERO = 0, NORM_DYT = 1 };

struct Layer {
    int type = 0;
    float *norm1 = nullptr, *norm2 = nullptr, *shift = nullptr;
    // rglru
    uint32_t C = 0, blocks = 0, taps = 0;
    Weight yx, gates, o;
    float *yx_b = nullptr, *conv = nullptr, *conv_b = nullptr, *gates_b = nullptr, *lam = nullptr;
    // latent attention
    uint32_t H = 0, dim = 0, vdim = 0, R = 0, QR = 0; float scale = 0.0f;
    Weight dqkv, uq, ukT, uv;
    float *dq_norm = nullptr, *dkv_norm = nullptr;
    // latent attention with direct queries (QR == 0): proj = [q | down-projection | gate]; RD rotated key columns beside the latent
    // (rot_dims of them turn, table rot_tab), RS the length of a cache row, window (kAttnNoWindow: causal), sink per head (optional),
    // has_gate: sigmoid(W_g h) multiplies the concatenated heads
    uint32_t RD = 0, RS = 0; float *sink = nullptr; bool has_gate = false;
    // hyper-connected form: layer norms of the two sublayers, their layer scales (optional) and connection weights [in | out | mix]
    float *ln1 = nullptr, *ln2 = nullptr, *ls1 = nullptr, *ls2 = nullptr, *hc1 = nullptr, *hc2 = nullptr;
    // sandwich form: input / output norms of the mixer and of the feed-forward
    float *n1 = nullptr, *n1b = nullptr, *n2 = nullptr, *n2b = nullptr;
    // retention: proj = [q | k | v | g]
    float *decay = nullptr; uint32_t rot_dims = 0; float2 *rot_tab = nullptr;
    Weight proj;
    // window attention + selective scan side by side: proj = [q | k | x | g | z]; H, dim as above, G key/value heads
    uint32_t G = 0, a_taps = 0, window = 0, RL = 0; float softcap = 0.0f, left_scale = 1.0f, right_scale = 1.0f;
    float *a_conv = nullptr, *temp = nullptr, *talk = nullptr, *slopes = nullptr;
    uint32_t mC = 0, mN = 0, mR = 0, m_taps = 0;
    float *m_conv = nullptr, *m_conv_b = nullptr, *dt_b = nullptr, *A = nullptr, *Dv = nullptr;
    Weight xw, dtw, mo; float *dt_wf = nullptr;      // dt_wf: the step-size projection once more in fp32, for the scan that makes dt itself
    // Dynamic-Tanh norms of the sequential form
    Dyt d1{}, d1b{}, d2{}, d2b{};
    // differential attention: proj = [q | k | v] with its biases (q alone when the keys and values are layer kv_from's); H, G, dim, vdim,
    // scale, rot_dims, rot_tab, RL as above; lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff
    int kv_from = -1; float diff = 0.0f, lambda = 0.0f; float *proj_b = nullptr, *o_b = nullptr;
    uint32_t a_hpb = 0, a_ngk = 0, a_qt = 0;      // heads per attention block, kv heads such a block stages, query tokens per prefill block
    uint32_t a_hpb1 = 0, a_ngk1 = 0;              // the same for short portions: blocks of one kv head's query heads, so that more blocks share the keys
    // state-space duality: proj = [z | x | B | C | dt]; H heads of vdim, mN states, G groups, m_taps, m_conv, m_conv_b, dt_b, A = exp(A_log)
    // per head, Dv per head; the output is normed in `parts` equal parts with the gain gn
    uint32_t parts = 0; float *gn = nullptr;
    // feed-forward
    int ff_kind = FF_NONE; float *act = nullptr;
    bool has_mlp = false, has_shared = false;
    // scored experts: how the router weighs (k_route's mode), whether the weight scales what the expert reads (else its output), whether
    // the shared expert sits behind a gate row of the router, the gated unit (k_gemv's glu) and its limits
    uint32_t route_mode = 1, glu_kind = 2; bool score_in = true, sh_gate = false; float limit = 0.0f, slimit = 0.0f;
    uint32_t NE = 0, top = 0, ff = 0, sff = 0;
    float *router = nullptr;
    Weight up, down, sup, sdown;
};

struct Run { uint32_t layer = 0; bool add_embed = false; size_t st_prev = 0, st_S = 0, st_conv = 0, st_conv2 = 0; float *cache = nullptr; };

struct Seq { bool live = false; uint32_t len = 0; std::vector<uint32_t> pages; };

constexpr float kRglruDecay = 8.0f;      // a = exp(-8 r softplus(lam)): fixed by the design
constexpr uint32_t kWantBatch = 64;      // rows of logits computed per head product
constexpr uint32_t kSplitMax = 32;
constexpr uint32_t kRetSegs = 8;             // time segments of a long retention portion (k_retention_chain holds as many states in registers)
constexpr uint32_t kNoWindow = 1u << 30;      // window of an attention without a mask: every earlier key is seen

}  // namespace

struct LayeredEngine : nb::EngineBase {
    int device = 0, num_sms = 148;
    cudaStream_t stream = nullptr, side = nullptr, side2 = nullptr, cur = nullptr;      // cur: where launch() puts kernels (stream, or side for a layer's feed-forward branch)
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr, ev_join2 = nullptr;
    bool f32 = false;
    uint32_t V = 0, E = 0; float eps = 0.0f;
    std::vector<Layer> layers; std::vector<Run> runs;
    bool keep_x0 = false;
    int form = FORM_PARALLEL_SHIFT;
    Weight embed, head, pos_table; float *final_norm = nullptr; uint32_t max_pos = 0;      // max_pos: rows of the position table (0: the design has none)
    // state manager
    uint32_t max_tokens = 0, max_seqs = 0, n_pages = 0, chunk_cap = 0; size_t slot_floats = 0;
    float *state = nullptr, *state_bak = nullptr; uint32_t *table = nullptr;
    std::vector<uint32_t> free_pages; std::vector<Seq> seqs;
    // scratch (chunk_cap tokens)
    float *x = nullptr, *x0 = nullptr, *hm = nullptr, *h2 = nullptr, *d = nullptr, *d2 = nullptr;
    float *b_yx = nullptr, *b_u = nullptr, *b_g = nullptr, *b_sy = nullptr;                          // recurrent block
    float *b_z = nullptr, *b_cq = nullptr, *b_q = nullptr, *b_qa = nullptr, *b_ol = nullptr, *b_ov = nullptr, *b_part = nullptr;   // attention
    float *b_wt = nullptr, *b_hb = nullptr, *b_eo = nullptr, *b_sh = nullptr, *b_so = nullptr;                   // feed-forward
    float *b_wpart = nullptr, *b_rseg = nullptr; uint32_t *b_wtick = nullptr, *b_rtick = nullptr;      // window attention: partials and tickets of the key splits
    float *b_p = nullptr, *b_qk = nullptr, *b_xc = nullptr, *b_a = nullptr, *b_ro = nullptr, *b_dbc = nullptr, *b_dt = nullptr, *b_y = nullptr, *b_f = nullptr;   // retention, window attention + selective scan, dense feed-forward
    uint32_t *b_tick = nullptr;      // attention: tickets of the key splits
    uint32_t *b_idx = nullptr, *b_cnt = nullptr, *b_off = nullptr, *b_fill = nullptr, *b_slot = nullptr, *b_rows = nullptr;
    float *b_xn = nullptr, *logits = nullptr, *keep = nullptr;
    // Dynamic-Tanh designs: embedding scale, the pair table and its hash, the norms around the stack, where a slot keeps the last token
    int norm_kind = NORM_RMS_ZERO; float emb_scale = 1.0f; Weight pairs; uint32_t buckets = 0, mul_prev = 0, mul_cur = 0; Dyt embed_norm{}, final_dyt{}; size_t st_tok = 0;
    std::vector<std::pair<std::string, float2 *>> rot_tabs;      // position tables of the rotary attention layers, one per distinct setting
    // short portions of a Dynamic-Tanh design: the residual update that follows a sublayer rides on the sublayer's last product
    struct ResEpi { bool on = false; Dyt post{}, pre{}; float *out = nullptr, *keep = nullptr; } res;
    float *b_dpart = nullptr, *b_sseg = nullptr, *b_sdx = nullptr, *b_sdy = nullptr, *b_f2 = nullptr, *b_hg = nullptr, *b_sh2 = nullptr, *b_sg = nullptr, *b_wrow = nullptr; uint32_t *b_dtick = nullptr;
    uint32_t *ids_dev = nullptr, *want_dev = nullptr, *next_dev = nullptr, *tok_host = nullptr; uint8_t *seen = nullptr;
    uint32_t last_T = 0;
    uint32_t S = 1; float res_mult = 1.0f; float *xs = nullptr;      // hyper-connected form: streams, the model's residual multiplier, the streams [S][chunk][E]
    uint32_t *dpos = nullptr, *zero_dev = nullptr;            // device-side position of a captured decode step; a constant 0
    bool branch_streams = true;      // a layer's feed-forward and shared expert on streams of their own (NB200_NO_BRANCH_STREAMS=1: one stream)
    bool use_pdl = true; bool use_graph = true; std::vector<cudaGraphExec_t> graphs; uint32_t graph_launches = 0;
    // generation on the implicit sequence
    int gen_seq = -1;
    void *samp_ws = nullptr; size_t samp_cub = 0; uint32_t *samp_host = nullptr;
    std::vector<void *> allocs;
};

namespace {

inline LayeredEngine *self(nb200_engine *e) { return reinterpret_cast<LayeredEngine *>(e); }
inline const LayeredEngine *self(const nb200_engine *e) { return reinterpret_cast<const LayeredEngine *>(e); }

int dmalloc(LayeredEngine *e, void **p, size_t bytes) {
    if (bytes == 0) bytes = 16;
    cudaError_t err = cudaMalloc(p, bytes);
    if (err != cudaSuccess) return fail(NB200_ENOMEM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(err));
    e->allocs.push_back(*p);
    return 0;
}
#define DM(ptr, bytes) do { int r_ = dmalloc(e, (void **)&(ptr), (bytes)); if (r_) return r_; } while (0)

// ---------------- loader ----------------
struct Loader {
    LayeredEngine *e; const nb::ModelDir *dir;

    int host_f32(const std::string &name, std::vector<float> *out, std::vector<uint64_t> *shape) {
        auto it = dir->tensors.find(name);
        if (it == dir->tensors.end()) return fail(NB200_EINVAL, "model.safetensors has no tensor \"%s\"", name.c_str());
        const nb::StTensor &t = it->second;
        const uint64_t n = t.count();
        out->resize(n);
        if (t.dtype == "BF16") {
            const uint16_t *s = reinterpret_cast<const uint16_t *>(t.data);
            for (uint64_t i = 0; i < n; i++) { const uint32_t u = (uint32_t)s[i] << 16; memcpy(&(*out)[i], &u, 4); }
        } else if (t.dtype == "F32") {
            memcpy(out->data(), t.data, n * 4);
        } else return fail(NB200_EINVAL, "tensor \"%s\" has dtype %s (BF16 or F32 expected)", name.c_str(), t.dtype.c_str());
        if (shape) *shape = t.shape;
        return 0;
    }
    int expect(const std::string &name, const std::vector<uint64_t> &got, std::initializer_list<uint64_t> want) {
        uint64_t n = 1;
        for (uint64_t v : got) n *= v;
        if (want.size() == 0 && n == 1) return 0;      // a single number, stored as [] or [1]
        if (got.size() != want.size() || !std::equal(got.begin(), got.end(), want.begin())) {
            std::string g, w;
            for (uint64_t v : got) g += std::to_string(v) + " ";
            for (uint64_t v : want) w += std::to_string(v) + " ";
            return fail(NB200_EINVAL, "tensor \"%s\" has shape [ %s] where the config implies [ %s]", name.c_str(), g.c_str(), w.c_str());
        }
        return 0;
    }
    // fp32 vector (norm gains, biases, taps, router): stays fp32 in every mode
    int vec(const std::string &name, std::initializer_list<uint64_t> shape, float **dst) {
        std::vector<float> h; std::vector<uint64_t> sh; int r;
        if ((r = host_f32(name, &h, &sh)) || (r = expect(name, sh, shape))) return r;
        return put_f32(h, dst);
    }
    int put_f32(const std::vector<float> &h, float **dst) {
        DM(*dst, h.size() * 4);
        CK(cudaMemcpy(*dst, h.data(), h.size() * 4, cudaMemcpyHostToDevice));
        e->weight_bytes += h.size() * 4;
        return 0;
    }
    // matrix in the compute type
    int put_w(const std::vector<float> &h, uint32_t rows, uint32_t cols, Weight *w) {
        w->rows = rows; w->cols = cols;
        if (e->f32) { float *p = nullptr; int r = put_f32(h, &p); w->p = p; return r; }
        std::vector<__nv_bfloat16> b(h.size());
        for (size_t i = 0; i < h.size(); i++) b[i] = __float2bfloat16_rn(h[i]);
        DM(w->p, b.size() * 2);
        CK(cudaMemcpy(w->p, b.data(), b.size() * 2, cudaMemcpyHostToDevice));
        e->weight_bytes += b.size() * 2;
        return 0;
    }
    // rows of several [r_i, cols] tensors stacked into one matrix
    int stacked(const std::vector<std::string> &names, const std::vector<uint64_t> &rows, uint64_t cols, Weight *w) {
        std::vector<float> all;
        uint64_t total = 0;
        for (size_t i = 0; i < names.size(); i++) {
            std::vector<float> h; std::vector<uint64_t> sh; int r;
            if ((r = host_f32(names[i], &h, &sh)) || (r = expect(names[i], sh, {rows[i], cols}))) return r;
            all.insert(all.end(), h.begin(), h.end());
            total += rows[i];
        }
        return put_w(all, (uint32_t)total, (uint32_t)cols, w);
    }
};

bool u32_of(const nb::Json *o, const char *key, uint32_t *v) {
    double d;
    if (!o || !o->number(key, &d) || d < 0 || d > 4294967295.0 || d != (double)(uint64_t)d) return false;
    *v = (uint32_t)d;
    return true;
}

int load_rglru(Loader &ld, const nb::Json *m, const std::string &p, Layer *L, uint32_t E) {
    if (!u32_of(m, "width", &L->C) || !u32_of(m, "blocks", &L->blocks) || !u32_of(m, "conv", &L->taps))
        return fail(NB200_EINVAL, "%s: an rglru mixer needs width, blocks and conv", p.c_str());
    if (!L->C || !L->blocks || !L->taps || L->C % L->blocks) return fail(NB200_EINVAL, "%s: width %u / blocks %u / conv %u unusable", p.c_str(), L->C, L->blocks, L->taps);
    const uint64_t C = L->C, B = L->blocks, bs = C / B;
    int r;
    if ((r = ld.stacked({p + "y", p + "x"}, {C, C}, E, &L->yx))) return r;
    {
        std::vector<float> a, b; std::vector<uint64_t> sa, sb;
        if ((r = ld.host_f32(p + "y.b", &a, &sa)) || (r = ld.expect(p + "y.b", sa, {C})) || (r = ld.host_f32(p + "x.b", &b, &sb)) || (r = ld.expect(p + "x.b", sb, {C}))) return r;
        a.insert(a.end(), b.begin(), b.end());
        if ((r = ld.put_f32(a, &L->yx_b))) return r;
    }
    if ((r = ld.vec(p + "conv", {C, L->taps}, &L->conv)) || (r = ld.vec(p + "conv.b", {C}, &L->conv_b)) || (r = ld.vec(p + "lam", {C}, &L->lam))) return r;
    {   // [recurrence gate blocks | input gate blocks], each block [bs, bs]
        std::vector<float> a, b, ab, bb; std::vector<uint64_t> s;
        if ((r = ld.host_f32(p + "ra", &a, &s)) || (r = ld.expect(p + "ra", s, {B, bs, bs})) || (r = ld.host_f32(p + "ri", &b, &s)) || (r = ld.expect(p + "ri", s, {B, bs, bs})) ||
            (r = ld.host_f32(p + "ra.b", &ab, &s)) || (r = ld.expect(p + "ra.b", s, {B, bs})) || (r = ld.host_f32(p + "ri.b", &bb, &s)) || (r = ld.expect(p + "ri.b", s, {B, bs}))) return r;
        a.insert(a.end(), b.begin(), b.end());
        ab.insert(ab.end(), bb.begin(), bb.end());
        if ((r = ld.put_w(a, (uint32_t)(2 * C), (uint32_t)bs, &L->gates)) || (r = ld.put_f32(ab, &L->gates_b))) return r;
    }
    return ld.stacked({p + "o"}, {E}, C, &L->o);
}

int load_latent_attn(Loader &ld, const nb::Json *m, const std::string &p, Layer *L, uint32_t E) {
    double sc;
    if (!u32_of(m, "heads", &L->H) || !u32_of(m, "dim", &L->dim) || !u32_of(m, "vdim", &L->vdim) || !u32_of(m, "kv_rank", &L->R) || !u32_of(m, "q_rank", &L->QR) ||
        !m->number("scale", &sc))
        return fail(NB200_EINVAL, "%s: a latent_attention mixer needs heads, dim, vdim, kv_rank, q_rank and scale", p.c_str());
    L->scale = (float)sc; L->RS = L->R; L->window = kAttnNoWindow;
    if (!L->H || !L->dim || !L->vdim || !L->R || !L->QR) return fail(NB200_EINVAL, "%s: zero-sized attention", p.c_str());
    if (L->R > 512) return fail(NB200_EINVAL, "%s: kv_rank %u above 512 has no attention kernel", p.c_str(), L->R);
    const uint64_t H = L->H, D = L->dim, VD = L->vdim, R = L->R, QR = L->QR;
    int r;
    if ((r = ld.stacked({p + "dq", p + "dkv"}, {QR, R}, E, &L->dqkv)) || (r = ld.vec(p + "dq.norm", {QR}, &L->dq_norm)) || (r = ld.vec(p + "dkv.norm", {R}, &L->dkv_norm)) ||
        (r = ld.stacked({p + "uq"}, {H * D}, QR, &L->uq)) || (r = ld.stacked({p + "uv"}, {H * VD}, R, &L->uv)) || (r = ld.stacked({p + "o"}, {E}, H * VD, &L->o))) return r;
    std::vector<float> uk, t(H * R * D); std::vector<uint64_t> s;
    if ((r = ld.host_f32(p + "uk", &uk, &s)) || (r = ld.expect(p + "uk", s, {H * D, R}))) return r;
    for (uint64_t h = 0; h < H; h++)          // [H*dim, R] -> per head [R, dim]: absorbed query = q_h W_uk,h
        for (uint64_t dd = 0; dd < D; dd++)
            for (uint64_t k = 0; k < R; k++) t[(h * R + k) * D + dd] = uk[(h * D + dd) * R + k];
    return ld.put_w(t, (uint32_t)(H * R), (uint32_t)D, &L->ukT);
}

int load_moe(Loader &ld, const nb::Json *f, const std::string &p, Layer *L, uint32_t E) {
    const nb::Json *kind = f->get("kind");
    if (!kind || kind->t != nb::Json::Str || kind->str != "moe") return fail(NB200_EINVAL, "%s: feed-forward kind \"%s\" is not known", p.c_str(), kind && kind->t == nb::Json::Str ? kind->str.c_str() : "?");
    if (!u32_of(f->get("router"), "experts", &L->NE) || !u32_of(f->get("router"), "top", &L->top) || !u32_of(f->get("expert"), "ff", &L->ff))
        return fail(NB200_EINVAL, "%s: a moe feed-forward needs router.experts, router.top and expert.ff", p.c_str());
    if (!L->NE || !L->top || L->top > L->NE || !L->ff) return fail(NB200_EINVAL, "%s: experts %u / top %u / ff %u unusable", p.c_str(), L->NE, L->top, L->ff);
    L->has_mlp = true; L->ff_kind = FF_MOE;
    int r;
    if ((r = ld.vec(p + "router", {L->NE, E}, &L->router))) return r;
    std::vector<std::string> ups, downs; std::vector<uint64_t> ur, dr;
    for (uint32_t i = 0; i < L->NE; i++) { ups.push_back(p + "e" + std::to_string(i) + ".up"); downs.push_back(p + "e" + std::to_string(i) + ".down"); ur.push_back(L->ff); dr.push_back(E); }
    if ((r = ld.stacked(ups, ur, E, &L->up)) || (r = ld.stacked(downs, dr, L->ff, &L->down))) return r;
    if (f->present("shared")) {
        if (!u32_of(f->get("shared"), "ff", &L->sff) || !L->sff) return fail(NB200_EINVAL, "%s: shared.ff missing", p.c_str());
        L->has_shared = true;
        if ((r = ld.stacked({p + "shared.up"}, {L->sff}, E, &L->sup)) || (r = ld.stacked({p + "shared.down"}, {E}, L->sff, &L->sdown))) return r;
    }
    return 0;
}

// rows [first, first + count) of tensor `name` ([total, cols]) appended to *all
int append_rows(Loader &ld, const std::string &name, uint64_t total, uint64_t cols, uint64_t first, uint64_t count, std::vector<float> *all) {
    std::vector<float> h; std::vector<uint64_t> sh; int r;
    if ((r = ld.host_f32(name, &h, &sh)) || (r = ld.expect(name, sh, {total, cols}))) return r;
    all->insert(all->end(), h.begin() + first * cols, h.begin() + (first + count) * cols);
    return 0;
}

int load_retention(Loader &ld, const nb::Json *m, const std::string &p, Layer *L, uint32_t E, uint32_t max_pos) {
    const nb::Json *decay = m->get("decay");
    if (!u32_of(m, "heads", &L->H) || !u32_of(m, "dim", &L->dim) || !u32_of(m, "vdim", &L->vdim) || !decay || decay->t != nb::Json::Arr)
        return fail(NB200_EINVAL, "%s: a retention mixer needs heads, dim, vdim and the list decay", p.c_str());
    if (!L->H || !L->dim || !L->vdim || decay->arr.size() != L->H) return fail(NB200_EINVAL, "%s: heads %u / dim %u / vdim %u / %zu decays unusable", p.c_str(), L->H, L->dim, L->vdim, decay->arr.size());
    if (L->dim > 256) return fail(NB200_EINVAL, "%s: dim %u above 256 has no retention kernel", p.c_str(), L->dim);
    const uint64_t H = L->H, D = L->dim, VD = L->vdim;
    std::vector<float> dec(H);
    for (uint32_t h = 0; h < H; h++) { if (decay->arr[h].t != nb::Json::Num) return fail(NB200_EINVAL, "%s: decay[%u] is no number", p.c_str(), h); dec[h] = (float)decay->arr[h].num; }
    int r;
    if ((r = ld.put_f32(dec, &L->decay))) return r;
    if (m->present("rot")) {
        const nb::Json *rot = m->get("rot");
        double base;
        if (!u32_of(rot, "dims", &L->rot_dims) || !rot->number("base", &base) || L->rot_dims > L->dim || (L->rot_dims & 1u) || !(base > 0.0))
            return fail(NB200_EINVAL, "%s: rot needs an even dims <= dim and a base > 0", p.c_str());
        const uint32_t half = L->rot_dims / 2u;
        if (half) {
            if (!max_pos) return fail(NB200_EINVAL, "%s: rotary positions need the model's position count", p.c_str());
            std::vector<float> tab((size_t)max_pos * half * 2);
            for (uint32_t i = 0; i < half; i++) {
                const double f = pow(base, -2.0 * (double)i / (double)L->rot_dims);
                for (uint32_t q = 0; q < max_pos; q++) { const double a = (double)q * f; tab[((size_t)q * half + i) * 2] = (float)cos(a); tab[((size_t)q * half + i) * 2 + 1] = (float)sin(a); }
            }
            float *t = nullptr;
            if ((r = ld.put_f32(tab, &t))) return r;
            L->rot_tab = reinterpret_cast<float2 *>(t);
        }
    }
    if ((r = ld.stacked({p + "q", p + "k", p + "v", p + "g"}, {H * D, H * D, H * VD, H * VD}, E, &L->proj))) return r;
    return ld.stacked({p + "o"}, {E}, H * VD, &L->o);
}

int load_window_ssm(Loader &ld, const nb::Json *m, const std::string &p, Layer *L, uint32_t E) {
    const nb::Json *lf = m->get("left"), *rt = m->get("right");
    double ls, rs, sc;
    if (!lf || lf->t != nb::Json::Obj || !rt || rt->t != nb::Json::Obj || !m->number("left_scale", &ls) || !m->number("right_scale", &rs))
        return fail(NB200_EINVAL, "%s: a parallel mixer needs left, right, left_scale and right_scale", p.c_str());
    L->left_scale = (float)ls; L->right_scale = (float)rs;
    if (!u32_of(lf, "heads", &L->H) || !u32_of(lf, "kv_heads", &L->G) || !u32_of(lf, "dim", &L->dim) || !u32_of(lf, "vdim", &L->vdim) || !u32_of(lf, "conv", &L->a_taps) || !lf->number("scale", &sc))
        return fail(NB200_EINVAL, "%sleft: window attention needs heads, kv_heads, dim, vdim, conv and scale", p.c_str());
    L->scale = (float)sc;
    if (!L->H || !L->G || L->H % L->G || !L->dim || !L->a_taps) return fail(NB200_EINVAL, "%sleft: heads %u / kv_heads %u / dim %u / conv %u unusable", p.c_str(), L->H, L->G, L->dim, L->a_taps);
    if (L->vdim != L->dim) return fail(NB200_EINVAL, "%sleft: the values are the keys, so vdim %u must equal dim %u", p.c_str(), L->vdim, L->dim);
    if (L->H > 32 || L->dim > 256) return fail(NB200_EINVAL, "%sleft: more than 32 heads or dim above 256 has no window-attention kernel", p.c_str());
    L->window = kNoWindow;
    if (lf->present("mask")) {
        if (!u32_of(lf->get("mask"), "size", &L->window) || !L->window) return fail(NB200_EINVAL, "%sleft: mask.size must be a positive integer", p.c_str());
        L->window = std::min(L->window, kNoWindow);
    }
    if (lf->present("softcap")) { double c; if (!lf->number("softcap", &c) || !(c >= 0.0)) return fail(NB200_EINVAL, "%sleft: softcap must be a number >= 0", p.c_str()); L->softcap = (float)c; }
    if (!u32_of(rt, "inner", &L->mC) || !u32_of(rt, "state", &L->mN) || !u32_of(rt, "dt_rank", &L->mR) || !u32_of(rt, "conv", &L->m_taps) || !L->mC || !L->mN || !L->mR || !L->m_taps)
        return fail(NB200_EINVAL, "%sright: a selective scan needs inner, state, dt_rank and conv", p.c_str());
    if (L->mN > 128) return fail(NB200_EINVAL, "%sright: state %u above 128 has no scan kernel", p.c_str(), L->mN);
    const uint64_t H = L->H, G = L->G, D = L->dim, C = L->mC, N = L->mN, R = L->mR;
    L->RL = (uint32_t)((G * D + G + 3u) & ~(uint64_t)3u);
    int r;
    {   // one product for both sides: [q | k | x | g | z]
        std::vector<float> all;
        if ((r = append_rows(ld, p + "left.q", H * D, E, 0, H * D, &all)) || (r = append_rows(ld, p + "left.k", G * D, E, 0, G * D, &all)) ||
            (r = append_rows(ld, p + "right.in", 2 * C, E, 0, C, &all)) || (r = append_rows(ld, p + "left.g", H * D, E, 0, H * D, &all)) ||
            (r = append_rows(ld, p + "right.in", 2 * C, E, C, C, &all))) return r;
        if ((r = ld.put_w(all, (uint32_t)(2 * H * D + G * D + 2 * C), E, &L->proj))) return r;
    }
    {   // taps of q and of k, one channel range
        std::vector<float> taps;
        if ((r = append_rows(ld, p + "left.q.conv", H * D, L->a_taps, 0, H * D, &taps)) || (r = append_rows(ld, p + "left.k.conv", G * D, L->a_taps, 0, G * D, &taps)) ||
            (r = ld.put_f32(taps, &L->a_conv))) return r;
    }
    if ((r = ld.vec(p + "left.temp", {H}, &L->temp)) || (r = ld.vec(p + "left.talk", {H, H}, &L->talk)) || (r = ld.stacked({p + "left.o"}, {E}, H * D, &L->o))) return r;
    std::vector<float> sl(H);
    for (uint32_t h = 0; h < H; h++) sl[h] = (float)pow(2.0, -8.0 * (double)(h + 1) / (double)H);
    if ((r = ld.put_f32(sl, &L->slopes))) return r;
    if ((r = ld.vec(p + "right.conv", {C, L->m_taps}, &L->m_conv)) || (r = ld.vec(p + "right.conv.b", {C}, &L->m_conv_b)) || (r = ld.vec(p + "right.dt.b", {C}, &L->dt_b)) ||
        (r = ld.vec(p + "right.D", {C}, &L->Dv)) || (r = ld.stacked({p + "right.x"}, {R + 2 * N}, C, &L->xw)) || (r = ld.stacked({p + "right.dt"}, {C}, R, &L->dtw)) ||
        (r = ld.stacked({p + "right.o"}, {E}, C, &L->mo)) || (r = ld.vec(p + "right.dt", {C, R}, &L->dt_wf))) return r;
    std::vector<float> al; std::vector<uint64_t> sh;
    if ((r = ld.host_f32(p + "right.A_log", &al, &sh)) || (r = ld.expect(p + "right.A_log", sh, {C, N}))) return r;
    for (float &v : al) v = (float)-exp((double)v);          // A = -exp(A_log)
    return ld.put_f32(al, &L->A);
}

int load_dense(Loader &ld, const nb::Json *f, const std::string &p, Layer *L, uint32_t E) {
    if (!u32_of(f, "ff", &L->ff) || !L->ff) return fail(NB200_EINVAL, "%s: a dense feed-forward needs ff", p.c_str());
    L->has_mlp = true; L->ff_kind = FF_DENSE_POLY;
    int r;
    if ((r = ld.stacked({p + "up"}, {L->ff}, E, &L->up)) || (r = ld.stacked({p + "down"}, {E}, L->ff, &L->down))) return r;
    return ld.vec(p + "act", {4}, &L->act);
}

uint32_t env_u32(const char *name, uint32_t dflt) { const char *s = getenv(name); return (s && *s) ? (uint32_t)strtoul(s, nullptr, 10) : dflt; }

// Dynamic-Tanh norm `name`: gain, bias `name`.b, one number `name`.alpha
int load_dyt(Loader &ld, const std::string &name, uint32_t E, Dyt *n) {
    float *w = nullptr, *b = nullptr; std::vector<float> al; std::vector<uint64_t> sh; int r;
    if ((r = ld.vec(name, {E}, &w)) || (r = ld.vec(name + ".b", {E}, &b)) || (r = ld.host_f32(name + ".alpha", &al, &sh)) || (r = ld.expect(name + ".alpha", sh, {}))) return r;
    n->w = w; n->b = b; n->alpha = al[0];
    return 0;
}

// names[i] are vectors of lens[i] numbers; joined into one fp32 vector
int joined_vec(Loader &ld, const std::vector<std::string> &names, const std::vector<uint64_t> &lens, float **dst) {
    std::vector<float> all;
    for (size_t i = 0; i < names.size(); i++) {
        std::vector<float> h; std::vector<uint64_t> sh; int r;
        if ((r = ld.host_f32(names[i], &h, &sh)) || (r = ld.expect(names[i], sh, {lens[i]}))) return r;
        all.insert(all.end(), h.begin(), h.end());
    }
    return ld.put_f32(all, dst);
}

// (cos, sin) of position x frequency for `positions` positions, built in double.  f_i = base^(-2i/dims), rescaled by wavelength
// l = 2 pi / f when `scaling` {factor, low, high, original} is given: kept where l < original / high, divided by factor where
// l > original / low, and between the two blended, (1 - s) f / factor + s f with s = (original / l - low) / (high - low).
int rope_table(Loader &ld, const nb::Json *rot, const std::string &p, uint32_t dims, uint32_t positions, float2 **out) {
    double base, factor = 1.0, low = 0.0, high = 0.0, original = 0.0;
    if (!rot->number("base", &base) || !(base > 0.0)) return fail(NB200_EINVAL, "%s: rot needs a base > 0", p.c_str());
    const nb::Json *sc = rot->present("scaling") ? rot->get("scaling") : nullptr;
    if (sc && (!sc->number("factor", &factor) || !sc->number("low", &low) || !sc->number("high", &high) || !sc->number("original", &original) || !(factor > 0.0) || !(high > low) || !(original > 0.0)))
        return fail(NB200_EINVAL, "%s: rot.scaling needs factor > 0, low < high and original > 0", p.c_str());
    char key[160];
    snprintf(key, sizeof key, "%u/%.17g/%d/%.17g/%.17g/%.17g/%.17g", dims, base, sc ? 1 : 0, factor, low, high, original);
    for (auto &kv : ld.e->rot_tabs) if (kv.first == key) { *out = kv.second; return 0; }
    const uint32_t half = dims / 2u;
    const double two_pi = 6.283185307179586476925286766559;
    std::vector<float> tab((size_t)positions * half * 2);
    for (uint32_t i = 0; i < half; i++) {
        double f = pow(base, -2.0 * (double)i / (double)dims);
        if (sc) {
            const double wave = two_pi / f;
            if (wave > original / low) f = f / factor;
            else if (!(wave < original / high)) { const double sm = (original / wave - low) / (high - low); f = (1.0 - sm) * f / factor + sm * f; }
        }
        for (uint32_t q = 0; q < positions; q++) { const double a = (double)q * f; tab[((size_t)q * half + i) * 2] = (float)cos(a); tab[((size_t)q * half + i) * 2 + 1] = (float)sin(a); }
    }
    float *t = nullptr; int r;
    if ((r = ld.put_f32(tab, &t))) return r;
    *out = reinterpret_cast<float2 *>(t);
    ld.e->rot_tabs.emplace_back(key, *out);
    return 0;
}

constexpr size_t kDiffSmemMax = 200 * 1024;
// grouped-query differential attention; `layers` lets a layer with kv_from check the layer it reads
int load_diff_attn(Loader &ld, const nb::Json *m, const std::string &p, Layer *L, uint32_t E, uint32_t positions, const std::vector<Layer> &layers, uint32_t self_index) {
    double sc, diff;
    if (!u32_of(m, "heads", &L->H) || !u32_of(m, "kv_heads", &L->G) || !u32_of(m, "dim", &L->dim) || !u32_of(m, "vdim", &L->vdim) || !m->number("scale", &sc) || !m->number("diff", &diff))
        return fail(NB200_EINVAL, "%s: an attention mixer needs heads, kv_heads, dim, vdim, scale and diff", p.c_str());
    L->scale = (float)sc; L->diff = (float)diff;
    if (!L->H || !L->G || L->H % L->G || !L->dim || !L->vdim) return fail(NB200_EINVAL, "%s: heads %u / kv_heads %u / dim %u / vdim %u unusable", p.c_str(), L->H, L->G, L->dim, L->vdim);
    if (L->vdim > 256) return fail(NB200_EINVAL, "%s: vdim %u above 256 has no attention kernel", p.c_str(), L->vdim);
    const uint64_t H = L->H, G = L->G, D = L->dim, VD = L->vdim;
    int r;
    if (m->present("rot")) {
        const nb::Json *rot = m->get("rot");
        if (!u32_of(rot, "dims", &L->rot_dims) || L->rot_dims > L->dim || (L->rot_dims & 1u)) return fail(NB200_EINVAL, "%s: rot needs an even dims <= dim", p.c_str());
        if (L->rot_dims && (r = rope_table(ld, rot, p, L->rot_dims, positions, &L->rot_tab))) return r;
    }
    L->RL = (uint32_t)((G * 2 * D + G * VD + 3u) & ~(uint64_t)3u);
    if (m->present("kv_from")) {
        uint32_t j = 0;
        if (!u32_of(m, "kv_from", &j) || j >= self_index || layers[j].type != MIX_DIFF_ATTN || layers[j].kv_from >= 0)
            return fail(NB200_EINVAL, "%s: kv_from must name an earlier attention layer with keys and values of its own", p.c_str());
        const Layer &S = layers[j];
        if (S.G != L->G || S.dim != L->dim || S.vdim != L->vdim || S.rot_dims != L->rot_dims || S.rot_tab != L->rot_tab) return fail(NB200_EINVAL, "%s: layer %u's keys and values have another shape or rotation", p.c_str(), j);
        L->kv_from = (int)j;
        if ((r = ld.stacked({p + "q"}, {H * 2 * D}, E, &L->proj)) || (r = ld.vec(p + "q.b", {H * 2 * D}, &L->proj_b))) return r;
    } else if ((r = ld.stacked({p + "q", p + "k", p + "v"}, {H * 2 * D, G * 2 * D, G * VD}, E, &L->proj)) ||
               (r = joined_vec(ld, {p + "q.b", p + "k.b", p + "v.b"}, {H * 2 * D, G * 2 * D, G * VD}, &L->proj_b))) return r;
    {   // one number for the layer: exp(lq1 . lk1) - exp(lq2 . lk2) + diff
        std::vector<float> v[4]; std::vector<uint64_t> sh; const char *nm[4] = {"lq1", "lk1", "lq2", "lk2"};
        for (int i = 0; i < 4; i++) if ((r = ld.host_f32(p + nm[i], &v[i], &sh)) || (r = ld.expect(p + nm[i], sh, {D}))) return r;
        double s1 = 0.0, s2 = 0.0;
        for (uint64_t i = 0; i < D; i++) { s1 += (double)v[0][i] * v[1][i]; s2 += (double)v[2][i] * v[3][i]; }
        L->lambda = (float)(exp(s1) - exp(s2) + diff);
    }
    if ((r = ld.stacked({p + "o"}, {E}, H * VD, &L->o)) || (r = ld.vec(p + "o.b", {E}, &L->o_b))) return r;
    // the widest block (heads per block, query tokens per prefill block) whose key and value slices fit the shared memory
    const bool vec = diff_attn_vec(L->dim, L->vdim, (uint32_t)(H * 2 * D + (L->kv_from < 0 ? G * 2 * D + G * VD : 0)));
    for (uint32_t hpb = std::min<uint32_t>(8u, L->H); hpb >= 1u && !L->a_hpb; hpb = hpb / 2u) {
        const uint32_t ngk = diff_attn_ngk(L->H, L->G, hpb);
        for (uint32_t qt : {4u, 1u})          // four query tokens per prefill block: 128 registers, two blocks per SM (eight measured 10 % slower at one block per SM)
            if (diff_attn_smem(L->dim, L->vdim, ngk, qt, hpb, vec) <= kDiffSmemMax) { L->a_hpb = hpb; L->a_ngk = ngk; L->a_qt = qt; break; }
    }
    if (L->a_hpb) {
        const uint32_t rep_ = L->H / L->G;
        L->a_hpb1 = rep_ >= 2u ? std::min(L->a_hpb, rep_) : std::min(L->a_hpb, 4u);
        L->a_ngk1 = diff_attn_ngk(L->H, L->G, L->a_hpb1);
    }
    if (!L->a_hpb) return fail(NB200_EINVAL, "%s: one key page of a key/value head (%u + %u floats per key) does not fit the attention kernel's shared memory", p.c_str(), 2 * L->dim, L->vdim);
    return 0;
}

int load_ssd(Loader &ld, const nb::Json *m, const std::string &p, Layer *L, uint32_t E) {
    if (!u32_of(m, "heads", &L->H) || !u32_of(m, "vdim", &L->vdim) || !u32_of(m, "state", &L->mN) || !u32_of(m, "groups", &L->G) || !u32_of(m, "conv", &L->m_taps) || !u32_of(m, "norm_groups", &L->parts))
        return fail(NB200_EINVAL, "%s: a mamba2 mixer needs heads, vdim, state, groups, conv and norm_groups", p.c_str());
    if (!L->H || !L->vdim || !L->mN || !L->G || L->H % L->G || !L->m_taps || !L->parts || (L->H * L->vdim) % L->parts)
        return fail(NB200_EINVAL, "%s: heads %u / vdim %u / state %u / groups %u / conv %u / norm_groups %u unusable", p.c_str(), L->H, L->vdim, L->mN, L->G, L->m_taps, L->parts);
    if (L->mN > 256) return fail(NB200_EINVAL, "%s: state %u above 256 has no scan kernel", p.c_str(), L->mN);
    const uint64_t Hn = L->H, inner = Hn * L->vdim, XW = inner + 2ull * L->G * L->mN;
    int r;
    if ((r = ld.stacked({p + "in"}, {inner + XW + Hn}, E, &L->proj)) || (r = ld.vec(p + "conv", {XW, L->m_taps}, &L->m_conv)) || (r = ld.vec(p + "conv.b", {XW}, &L->m_conv_b)) ||
        (r = ld.vec(p + "dt_bias", {Hn}, &L->dt_b)) || (r = ld.vec(p + "D", {Hn}, &L->Dv)) || (r = ld.vec(p + "norm", {inner}, &L->gn)) || (r = ld.stacked({p + "o"}, {E}, inner, &L->o))) return r;
    std::vector<float> al; std::vector<uint64_t> sh;
    if ((r = ld.host_f32(p + "A_log", &al, &sh)) || (r = ld.expect(p + "A_log", sh, {Hn}))) return r;
    for (float &v : al) v = (float)exp((double)v);          // the decay rate of a head: a_t = exp(-rate dt_t)
    return ld.put_f32(al, &L->A);
}

// gated feed-forward down(act(gate h) x (up h)): up = [gate | up] stacked
int load_glu_dense(Loader &ld, const nb::Json *f, const std::string &p, Layer *L, uint32_t E) {
    if (!u32_of(f, "ff", &L->ff) || !L->ff) return fail(NB200_EINVAL, "%s: a dense feed-forward needs ff", p.c_str());
    L->has_mlp = true; L->ff_kind = FF_DENSE_GLU;
    int r;
    if ((r = ld.stacked({p + "gate", p + "up"}, {L->ff, L->ff}, E, &L->up))) return r;
    return ld.stacked({p + "down"}, {E}, L->ff, &L->down);
}

// mixture of gated silu experts chosen by sigmoid scores; the router matrix carries the shared expert's gate as one more row
// clamped: the experts are clamped gated units with expert.limit / shared.limit, chosen by softmax scores over all experts that weigh
// their OUTPUT, and the shared expert has no gate
int load_moe_scored(Loader &ld, const nb::Json *f, const std::string &p, Layer *L, uint32_t E, bool clamped = false) {
    if (!u32_of(f->get("router"), "experts", &L->NE) || !u32_of(f->get("router"), "top", &L->top) || !u32_of(f->get("expert"), "ff", &L->ff))
        return fail(NB200_EINVAL, "%s: a moe feed-forward needs router.experts, router.top and expert.ff", p.c_str());
    if (!L->NE || !L->top || L->top > L->NE || !L->ff) return fail(NB200_EINVAL, "%s: experts %u / top %u / ff %u unusable", p.c_str(), L->NE, L->top, L->ff);
    L->has_mlp = true; L->ff_kind = FF_MOE_SCORED;
    int r;
    if (f->present("shared")) {
        if (!u32_of(f->get("shared"), "ff", &L->sff) || !L->sff) return fail(NB200_EINVAL, "%s: shared.ff missing", p.c_str());
        L->has_shared = true; L->sh_gate = !clamped;
        if ((r = ld.stacked({p + "shared.gate", p + "shared.up"}, {L->sff, L->sff}, E, &L->sup)) || (r = ld.stacked({p + "shared.down"}, {E}, L->sff, &L->sdown))) return r;
    }
    if (clamped) {
        double lim = 0.0, slim = 0.0;
        if (!f->get("expert")->number("limit", &lim) || (L->has_shared && !f->get("shared")->number("limit", &slim))) return fail(NB200_EINVAL, "%s: clamped experts need expert.limit (and shared.limit)", p.c_str());
        L->limit = (float)lim; L->slimit = (float)slim; L->route_mode = 2; L->glu_kind = 3; L->score_in = false;
    }
    {
        std::vector<float> all;
        if ((r = append_rows(ld, p + "router", L->NE, E, 0, L->NE, &all)) || (L->sh_gate && (r = append_rows(ld, p + "shared.sg", 1, E, 0, 1, &all))) || (r = ld.put_f32(all, &L->router))) return r;
    }
    std::vector<std::string> ups, downs; std::vector<uint64_t> ur, dr;
    for (uint32_t i = 0; i < L->NE; i++) {
        const std::string ep = p + "e" + std::to_string(i) + ".";
        ups.push_back(ep + "gate"); ups.push_back(ep + "up"); ur.push_back(L->ff); ur.push_back(L->ff);
        downs.push_back(ep + "down"); dr.push_back(E);
    }
    if ((r = ld.stacked(ups, ur, E, &L->up)) || (r = ld.stacked(downs, dr, L->ff, &L->down))) return r;
    return 0;
}

// latent attention with direct queries: q = W_q h laid out per head as [dim | rot_dim]; the down-projection gives the latent (kv_rank
// rows, RMS-normed with a vector gain) and rot_dim more rows, one rotated key part for all heads.  Optional by presence: rot_dim / rot,
// mask.size (sliding window), the tensor sink (one more term in the softmax denominator per head), the tensor g (sigmoid output gate).
int load_latent_attn_direct(Loader &ld, const nb::Json *m, const std::string &p, Layer *L, uint32_t E, uint32_t positions) {
    double sc;
    if (!u32_of(m, "heads", &L->H) || !u32_of(m, "dim", &L->dim) || !u32_of(m, "vdim", &L->vdim) || !u32_of(m, "kv_rank", &L->R) || !m->number("scale", &sc))
        return fail(NB200_EINVAL, "%s: a latent attention mixer needs heads, dim, vdim, kv_rank and scale", p.c_str());
    L->scale = (float)sc; L->QR = 0;
    if (m->present("rot_dim") && !u32_of(m, "rot_dim", &L->RD)) return fail(NB200_EINVAL, "%s: rot_dim must be a non-negative integer", p.c_str());
    if (!L->H || !L->dim || !L->vdim || !L->R) return fail(NB200_EINVAL, "%s: zero-sized attention", p.c_str());
    if (L->R > 512) return fail(NB200_EINVAL, "%s: kv_rank %u above 512 has no attention kernel", p.c_str(), L->R);
    int r;
    if (L->RD && m->present("rot")) {
        const nb::Json *rot = m->get("rot");
        if (!u32_of(rot, "dims", &L->rot_dims) || L->rot_dims > L->RD || (L->rot_dims & 1u)) return fail(NB200_EINVAL, "%s: rot needs an even dims <= rot_dim", p.c_str());
        if (L->rot_dims && (r = rope_table(ld, rot, p, L->rot_dims, positions, &L->rot_tab))) return r;
    }
    L->window = kAttnNoWindow;
    if (m->present("mask")) {
        if (!u32_of(m->get("mask"), "size", &L->window) || !L->window) return fail(NB200_EINVAL, "%s: mask.size must be a positive integer", p.c_str());
        L->window = std::min(L->window, kAttnNoWindow);
    }
    const uint64_t H = L->H, D = L->dim, VD = L->vdim, R = L->R, RD = L->RD;
    L->RS = (uint32_t)((R + RD + 3u) & ~(uint64_t)3u);
    L->has_gate = ld.dir->tensors.count(p + "g") != 0;
    if (L->has_gate) r = ld.stacked({p + "q", p + "dkv", p + "g"}, {H * (D + RD), R + RD, H * VD}, E, &L->proj);
    else r = ld.stacked({p + "q", p + "dkv"}, {H * (D + RD), R + RD}, E, &L->proj);
    if (r || (r = ld.vec(p + "dkv.norm", {R}, &L->dkv_norm)) || (r = ld.stacked({p + "uv"}, {H * VD}, R, &L->uv)) || (r = ld.stacked({p + "o"}, {E}, H * VD, &L->o))) return r;
    if (ld.dir->tensors.count(p + "sink") && (r = ld.vec(p + "sink", {H}, &L->sink))) return r;
    std::vector<float> uk, t(H * R * D); std::vector<uint64_t> s;
    if ((r = ld.host_f32(p + "uk", &uk, &s)) || (r = ld.expect(p + "uk", s, {H * D, R}))) return r;
    for (uint64_t h = 0; h < H; h++)          // [H*dim, R] -> per head [R, dim]: absorbed query = q_h W_uk,h
        for (uint64_t dd = 0; dd < D; dd++)
            for (uint64_t k = 0; k < R; k++) t[(h * R + k) * D + dd] = uk[(h * D + dd) * R + k];
    return ld.put_w(t, (uint32_t)(H * R), (uint32_t)D, &L->ukT);
}

// dense feed-forward down(gelu(up h)) with the exact (erf) gelu
int load_dense_gelu(Loader &ld, const nb::Json *f, const std::string &p, Layer *L, uint32_t E) {
    if (!u32_of(f, "ff", &L->ff) || !L->ff) return fail(NB200_EINVAL, "%s: a dense feed-forward needs ff", p.c_str());
    L->has_mlp = true; L->ff_kind = FF_DENSE_GELU;
    int r;
    if ((r = ld.stacked({p + "up"}, {L->ff}, E, &L->up))) return r;
    return ld.stacked({p + "down"}, {E}, L->ff, &L->down);
}

// connection weights of one sublayer, packed [in S | out S | mix S x S (from, to)]; without the tensors a single stream is the plain residual
int load_hc(Loader &ld, const std::string &p, uint32_t S, float **dst) {
    std::vector<float> all;
    if (!ld.dir->tensors.count(p + "in")) {
        if (S != 1) return fail(NB200_EINVAL, "%s: %u residual streams need the tensors %sin, %sout and %smix", p.c_str(), S, p.c_str(), p.c_str(), p.c_str());
        all = {1.0f, 1.0f, 1.0f};
        return ld.put_f32(all, dst);
    }
    std::vector<float> h; std::vector<uint64_t> sh; int r;
    if ((r = ld.host_f32(p + "in", &h, &sh)) || (r = ld.expect(p + "in", sh, {S}))) return r;
    all.insert(all.end(), h.begin(), h.end());
    if ((r = ld.host_f32(p + "out", &h, &sh)) || (r = ld.expect(p + "out", sh, {S}))) return r;
    all.insert(all.end(), h.begin(), h.end());
    if ((r = ld.host_f32(p + "mix", &h, &sh)) || (r = ld.expect(p + "mix", sh, {S, S}))) return r;
    all.insert(all.end(), h.begin(), h.end());
    return ld.put_f32(all, dst);
}

// ---------------- launches ----------------
template <typename A>
int launch(LayeredEngine *e, void (*k)(const A), dim3 grid, dim3 block, size_t smem, const A &args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = e->cur;
    cudaLaunchAttribute attr[1];
    if (e->use_pdl) {      // programmatic dependent launch: see pdl_enter() in layered_kernels.cuh
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr; cfg.numAttrs = 1;
    }
    CK(cudaLaunchKernelEx(&cfg, k, args));
    e->launches++;
    return 0;
}

uint32_t gemv_blocks(const LayeredEngine *e, uint32_t N, uint32_t groups) {
    return std::min((N + 7u) / 8u, std::max(1u, (uint32_t)e->num_sms * 8u / groups));
}

// one matrix product; maxM = the most rows any group can have.  wf32: the weights are fp32 whatever the engine's mode (router).
// active: how many of the groups can have rows at all (routed products: tokens x top); the matrix-vector grid is sized for those
int gemm(LayeredEngine *e, GemmArgs a, uint32_t groups, uint32_t maxM, bool wf32 = false, uint32_t active = 0) {
    if (!a.a_gmod) a.a_gmod = 1;
    const bool f32 = e->f32 || wf32;
    if (maxM <= kGemvMaxM) {
        a.round_a = f32 ? 0u : 1u;
        const uint32_t gx = gemv_blocks(e, a.N, active ? std::min(active, groups) : groups);
        if (a.epi == EPI_CONV_RANGES)
            return f32 ? launch<GemmArgs>(e, k_gemv_ext<float, 1>, dim3(gx, groups), dim3(256), 0, a) : launch<GemmArgs>(e, k_gemv_ext<__nv_bfloat16, 1>, dim3(gx, groups), dim3(256), 0, a);
        if (a.res_x && a.a_parts <= 1)
            return f32 ? launch<GemmArgs>(e, k_gemv_ext<float, 5>, dim3(gx, groups), dim3(256), 0, a) : launch<GemmArgs>(e, k_gemv_ext<__nv_bfloat16, 5>, dim3(gx, groups), dim3(256), 0, a);
        if (a.a_parts > 1)
            return f32 ? launch<GemmArgs>(e, k_gemv_ext<float, 4>, dim3(gx, groups), dim3(256), 0, a) : launch<GemmArgs>(e, k_gemv_ext<__nv_bfloat16, 4>, dim3(gx, groups), dim3(256), 0, a);
        if (a.glu)
            return f32 ? launch<GemmArgs>(e, k_gemv_ext<float, 3>, dim3(gx, groups), dim3(256), 0, a) : launch<GemmArgs>(e, k_gemv_ext<__nv_bfloat16, 3>, dim3(gx, groups), dim3(256), 0, a);
        if (a.a_poly)
            return f32 ? launch<GemmArgs>(e, k_gemv_ext<float, 2>, dim3(gx, groups), dim3(256), 0, a) : launch<GemmArgs>(e, k_gemv_ext<__nv_bfloat16, 2>, dim3(gx, groups), dim3(256), 0, a);
        return f32 ? launch<GemmArgs>(e, k_gemv<float>, dim3(gx, groups), dim3(256), 0, a) : launch<GemmArgs>(e, k_gemv<__nv_bfloat16>, dim3(gx, groups), dim3(256), 0, a);
    }
    if (a.glu) return fail(NB200_EINVAL, "the gated-pair product is a matrix-vector instance (portions of at most %u tokens)", kGemvMaxM);
    const dim3 grid((a.N + 63u) / 64u, (maxM + 63u) / 64u, groups);
    return f32 ? launch<GemmArgs>(e, k_gemm_f32<float>, grid, dim3(256), 0, a) : launch<GemmArgs>(e, k_gemm_bf16, grid, dim3(128), 0, a);
}

GemmArgs plain(const float *A, uint32_t lda, const Weight &w, float *C, uint32_t ldc, uint32_t M, const float *bias = nullptr, uint32_t epi = EPI_NONE, uint32_t split = 0) {
    GemmArgs a{};
    a.A = A; a.lda = lda; a.W = w.p; a.ldw = w.cols; a.C = C; a.ldc = ldc; a.M = M; a.N = w.rows; a.K = w.cols; a.bias = bias;
    a.epi = bias && epi == EPI_NONE ? EPI_BIAS : epi; a.split = split; a.a_gmod = 1;
    return a;
}

uint32_t ew_grid(size_t n) { return (uint32_t)std::min<size_t>((n + 255) / 256, 148 * 16); }

constexpr int kAttnQT = 8;      // query tokens per attention block in a prefill portion (4 where the latent is wider than 256)
size_t attn_smem(uint32_t R, int qt) { return ((size_t)qt * kAttnWarps * R + (size_t)kPage * (R + 4)) * 4; }

template <int RCH, int QT>
int attn_launch_r(LayeredEngine *e, const AttnArgs &a, dim3 grid, dim3 block, size_t smem) {
    if (a.KX || a.window < kAttnNoWindow || a.sink)      // the instance with the options
        return a.R == (uint32_t)RCH * 32u ? launch<AttnArgs>(e, k_latent_attn<RCH, QT, true, true>, grid, block, smem, a) : launch<AttnArgs>(e, k_latent_attn<RCH, QT, false, true>, grid, block, smem, a);
    return a.R == (uint32_t)RCH * 32u ? launch<AttnArgs>(e, k_latent_attn<RCH, QT, true>, grid, block, smem, a) : launch<AttnArgs>(e, k_latent_attn<RCH, QT, false>, grid, block, smem, a);
}
template <int QT>
int attn_launch_qt(LayeredEngine *e, const AttnArgs &a, uint32_t rch) {
    const dim3 grid((a.T + QT - 1) / QT, a.nsplit, (a.H + kAttnWarps - 1) / kAttnWarps), block(kAttnWarps * 32);
    const size_t smem = attn_smem(a.R + a.KX, QT);
    if (rch <= 2) return attn_launch_r<2, QT>(e, a, grid, block, smem);
    if (rch <= 4) return attn_launch_r<4, QT>(e, a, grid, block, smem);
    if (rch <= 8) return attn_launch_r<8, QT>(e, a, grid, block, smem);
    return attn_launch_r<16, QT>(e, a, grid, block, smem);
}
int attn_launch(LayeredEngine *e, const AttnArgs &a, uint32_t rch) {
    if (a.T <= kGemvMaxM) return attn_launch_qt<1>(e, a, rch);
    return rch <= 8 ? attn_launch_qt<kAttnQT>(e, a, rch) : attn_launch_qt<4>(e, a, rch);
}
template <int RCH, int QT>
int attn_optin_r(int smem) {
    CK(cudaFuncSetAttribute((const void *)k_latent_attn<RCH, QT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_latent_attn<RCH, QT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_latent_attn<RCH, QT, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_latent_attn<RCH, QT, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    return 0;
}
template <int QT>
int attn_optin(int smem) {
    int r;
    if ((r = attn_optin_r<2, QT>(smem)) || (r = attn_optin_r<4, QT>(smem)) || (r = attn_optin_r<8, QT>(smem)) || (r = attn_optin_r<16, QT>(smem))) return r;
    return 0;
}

// ---------------- mixers: e->hm [T][E] -> e->d [T][E], from the cache pages and the state slot of the sequence ----------------
struct Ctx { float *st; const uint32_t *table; uint32_t T, pos0; const uint32_t *pos_ptr; };

int mix_rglru(LayeredEngine *e, const Layer &L, const Run &run, const Ctx &cx) {
    const uint32_t E = e->E, T = cx.T; float *st = cx.st; int r;
    const uint32_t C = L.C, bs = C / L.blocks;
    if (T <= kGemvMaxM) {
        // short portions: the convolution is the epilogue of the [y | x] product, gates and recurrence are one kernel
        GemmArgs yx = plain(e->hm, E, L.yx, e->b_yx, 2 * C, T, L.yx_b, EPI_GELU_CONV, C);
        yx.cv_taps = L.conv; yx.cv_bias = L.conv_b; yx.cv_state = st + run.st_conv; yx.cv_out = e->b_u; yx.cv_K = L.taps;
        if ((r = gemm(e, yx, 1, T))) return r;
        GatesScanArgs gs{e->b_u, L.gates.p, L.gates_b, e->b_yx, 2 * C, L.lam, st + run.st_S, e->b_sy, T, C, bs, kRglruDecay, e->f32 ? 0u : 1u};
        const dim3 grid((C + 7u) / 8u), block(256);
        if ((r = e->f32 ? launch<GatesScanArgs>(e, k_rglru_gates_scan<float>, grid, block, 0, gs) : launch<GatesScanArgs>(e, k_rglru_gates_scan<__nv_bfloat16>, grid, block, 0, gs))) return r;
    } else {
        if ((r = gemm(e, plain(e->hm, E, L.yx, e->b_yx, 2 * C, T, L.yx_b, EPI_GELU_SPLIT, C), 1, T))) return r;
        ConvArgs ca{e->b_yx + C, 2 * C, L.conv, L.conv_b, st + run.st_conv, e->b_u, T, C, L.taps};
        if ((r = launch<ConvArgs>(e, k_conv, dim3(ew_grid((size_t)T * C)), dim3(256), 0, ca))) return r;
        if (L.taps > 1 && (r = launch<ConvArgs>(e, k_conv_state, dim3((C + 127) / 128), dim3(128), 0, ca))) return r;
        GemmArgs g{};
        g.A = e->b_u; g.lda = C; g.W = L.gates.p; g.ldw = bs; g.C = e->b_g; g.ldc = 2 * C; g.bias = L.gates_b; g.M = T; g.N = bs; g.K = bs;
        g.a_gmod = L.blocks; g.a_gcols = bs; g.c_gcols = bs; g.b_gstride = bs; g.w_gstride = (uint64_t)bs * bs; g.epi = EPI_SIGMOID;
        if ((r = gemm(e, g, 2 * L.blocks, T))) return r;
        ScanArgs sa{e->b_g, 2 * C, e->b_u, e->b_yx, 2 * C, L.lam, st + run.st_S, e->b_sy, T, C, kRglruDecay};
        if (T <= 32) { if ((r = launch<ScanArgs>(e, k_rglru_scan, dim3((C + 63) / 64), dim3(64), 0, sa))) return r; }
        else if ((r = launch<ScanArgs>(e, k_rglru_scan_par, dim3((C + 31) / 32), dim3(32, T >= 256 ? 32 : 8), 0, sa))) return r;
    }
    if ((r = gemm(e, plain(e->b_sy, C, L.o, e->d, E, T), 1, T))) return r;
    return 0;
}

int mix_latent_attn(LayeredEngine *e, const Layer &L, const Run &run, const Ctx &cx) {
    const uint32_t E = e->E, T = cx.T, pos0 = cx.pos0; const uint32_t *table = cx.table, *pos_ptr = cx.pos_ptr; int r;
    const uint32_t H = L.H, R = L.R, QR = L.QR, RS = L.RS;
    GemmArgs g{};      // absorb: qa[t][h][0..R) = q[t][h] W_uk,h
    g.W = L.ukT.p; g.ldw = L.dim; g.C = e->b_qa; g.ldc = H * RS; g.M = T; g.N = R; g.K = L.dim;
    g.a_gmod = H; g.c_gcols = RS; g.w_gstride = (uint64_t)R * L.dim;
    const uint32_t QW = H * (L.dim + L.RD), ZW = R + L.RD, P = QW + ZW + (L.has_gate ? H * L.vdim : 0u);      // direct queries: columns of the joint product
    if (QR) {      // queries through a normed latent of their own
        if ((r = gemm(e, plain(e->hm, E, L.dqkv, e->b_z, QR + R, T), 1, T))) return r;
        LatentNormArgs na{e->b_z, QR + R, L.dq_norm, L.dkv_norm, e->b_cq, run.cache, table, QR, R, pos0, e->eps, pos_ptr};
        if (T <= kGemvMaxM) {      // the norms ride on the query up-projection
            GemvLatentArgs ga{plain(e->b_z, QR + R, L.uq, e->b_q, H * L.dim, T), na, T};
            ga.g.a_norm_w = L.dq_norm; ga.g.a_eps = e->eps; ga.g.round_a = e->f32 ? 0u : 1u;
            const dim3 grid(gemv_blocks(e, ga.g.N, 1)), block(256);
            if ((r = e->f32 ? launch<GemvLatentArgs>(e, k_gemv_latent<float>, grid, block, 0, ga) : launch<GemvLatentArgs>(e, k_gemv_latent<__nv_bfloat16>, grid, block, 0, ga))) return r;
        } else {
            if ((r = launch<LatentNormArgs>(e, k_latent_norm, dim3(T), dim3(128), 0, na))) return r;
            if ((r = gemm(e, plain(e->b_cq, QR, L.uq, e->b_q, H * L.dim, T), 1, T))) return r;
        }
        g.A = e->b_q; g.lda = H * L.dim; g.a_gcols = L.dim;
        if ((r = gemm(e, g, H, T))) return r;
    } else {
        // one product gives [q | down-projection | gate]; the latent's norm, both rotations and the cache write are one kernel, for
        // short portions the last block of the absorb product
        if ((r = gemm(e, plain(e->hm, E, L.proj, e->b_z, P, T, nullptr, L.has_gate ? EPI_SIGMOID_TAIL : EPI_NONE, QW + ZW), 1, T))) return r;
        LatentRopeArgs ra{e->b_z, P, 0u, QW, L.dkv_norm, run.cache, table, e->b_qa, T, H, L.dim, L.RD, R, RS, L.rot_dims, L.rot_tab, pos0, e->eps, pos_ptr};
        g.A = e->b_z; g.lda = P; g.a_gcols = L.dim + L.RD;
        if (T <= kGemvMaxM) {
            GemvLatentRopeArgs ga{g, ra};
            ga.g.round_a = e->f32 ? 0u : 1u;
            const dim3 grid(gemv_blocks(e, g.N, H), H), block(256);
            if ((r = e->f32 ? launch<GemvLatentRopeArgs>(e, k_gemv_latent_rope<float>, grid, block, 0, ga) : launch<GemvLatentRopeArgs>(e, k_gemv_latent_rope<__nv_bfloat16>, grid, block, 0, ga))) return r;
        } else if ((r = launch<LatentRopeArgs>(e, k_latent_rope, dim3(T), dim3(128), 0, ra)) || (r = gemm(e, g, H, T))) return r;
    }
    AttnArgs aa{e->b_qa, run.cache, table, e->b_ol, e->b_part, T, H, R, pos0, 1u, L.scale, pos_ptr, e->b_tick, RS - R, L.window, L.sink};
    if (T <= kGemvMaxM) {      // short portions: the key pages in sight are dealt out to several blocks (two pages each at least)
        // a captured step does not know the position: the most pages a window can span; splits without keys write empty partials
        const uint32_t reach = pos_ptr ? e->max_tokens : pos0 + T;
        const uint32_t pages = (std::min(reach, L.window + T) + kPage - 1) / kPage;
        aa.nsplit = std::max(1u, std::min(kSplitMax, pos_ptr ? (pages + 2u) / 2u : pages / 2u));      // a window that starts inside a page spans one page more
    }
    if ((r = attn_launch(e, aa, (R + 31) / 32))) return r;
    GemmArgs v{};      // values: ov[t][h] = W_uv,h ol[t][h], times the output gate where the design has one
    v.A = e->b_ol; v.lda = H * R; v.W = L.uv.p; v.ldw = R; v.C = e->b_ov; v.ldc = H * L.vdim; v.M = T; v.N = L.vdim; v.K = R;
    v.a_gmod = H; v.a_gcols = R; v.c_gcols = L.vdim; v.w_gstride = (uint64_t)L.vdim * R;
    if (!QR && L.has_gate) { v.mul = e->b_z + QW + ZW; v.ldm = P; }
    if ((r = gemm(e, v, H, T))) return r;
    if ((r = gemm(e, plain(e->b_ov, H * L.vdim, L.o, e->d, E, T), 1, T))) return r;
    return 0;
}

// retention: [q | k | v | g] in one product; the scan rotates q and k while it stages them (k scaled by dim^-1/2 afterwards) and runs
// the recurrence over the fp32 state of the slot; per-head unit RMS times silu(g); output product
int mix_retention(LayeredEngine *e, const Layer &L, const Run &run, const Ctx &cx) {
    const uint32_t E = e->E, T = cx.T, H = L.H, D = L.dim, VD = L.vdim, P = 2 * H * D + 2 * H * VD;
    int r;
    if ((r = gemm(e, plain(e->hm, E, L.proj, e->b_p, P, T), 1, T))) return r;
    const bool small = T <= kGemvMaxM;      // short portions: the last block of a head also norms and gates its output
    RetentionArgs sa{e->b_p, P, 0, H * D, 2 * H * D, L.decay, cx.st + run.st_S, e->b_ro, T, H, D, VD,
                     L.rot_dims, cx.pos0, L.rot_tab, (float)(1.0 / sqrt((double)D)), cx.pos_ptr,
                     small ? 1u : 0u, e->b_p + 2 * H * D + H * VD, P, e->b_a, e->eps, e->b_rtick, 0u, 0u, e->b_rseg};
    // long portions: time segments side by side (built states, chained, then replayed with outputs)
    const uint32_t nseg = T >= 64 ? std::min(kRetSegs, T / 32u) : 1u;
    if (nseg > 1) {
        // every block of a head stages the head's q and k: rotate them once, in place, instead of in each of those blocks
        sa.seg_len = (T + nseg - 1u) / nseg;
        RopeArgs ra{e->b_p, P, 0, H * D, T, H, D, L.rot_dims, cx.pos0, L.rot_tab, sa.kscale, cx.pos_ptr};
        if ((r = launch<RopeArgs>(e, k_rope, dim3(ew_grid((size_t)T * H * (D - (L.rot_tab ? L.rot_dims / 2u : 0u)))), dim3(256), 0, ra))) return r;
        sa.rot_tab = nullptr; sa.kscale = 1.0f;
    }
    // columns per warp: four (fewest staged bytes per FMA) where the grid still gives every SM a dozen warps, else one
    const uint32_t cpw = (size_t)H * VD / 4u * nseg >= (size_t)e->num_sms * 12u ? 4u : 1u;
    const dim3 grid((VD + 8u * cpw - 1u) / (8u * cpw), H, nseg), block(256);
    for (uint32_t pass = (nseg > 1 ? 1u : 0u); pass <= (nseg > 1 ? 2u : 0u); pass++) {
        sa.mode = pass;
#define RET_LAUNCH(DCH) (cpw == 4 ? launch<RetentionArgs>(e, k_retention_scan<DCH, 4>, grid, block, 0, sa) : launch<RetentionArgs>(e, k_retention_scan<DCH, 1>, grid, block, 0, sa))
        if (D <= 32) r = RET_LAUNCH(1);
        else if (D <= 64) r = RET_LAUNCH(2);
        else if (D <= 128) r = RET_LAUNCH(4);
        else r = RET_LAUNCH(8);
#undef RET_LAUNCH
        if (r) return r;
        if (pass == 1) {
            RetChainArgs ca{cx.st + run.st_S, e->b_rseg, L.decay, H, D, VD, T, sa.seg_len, nseg};
            if ((r = launch<RetChainArgs>(e, k_retention_chain, dim3((VD * D + 255u) / 256u, H), dim3(256), 0, ca))) return r;
        }
    }
    if (r) return r;
    if (!small) {
        RetOutArgs oa{e->b_ro, e->b_p + 2 * H * D + H * VD, P, e->b_a, T, H, VD, e->eps};
        if ((r = launch<RetOutArgs>(e, k_retention_out, dim3((T * H + 7u) / 8u), dim3(256), 0, oa))) return r;
    }
    return gemm(e, plain(e->b_a, H * VD, L.o, e->d, E, T), 1, T);
}

template <int VCH>
int win_attn_launch_v(LayeredEngine *e, const WinAttnArgs &a, uint32_t qt, uint32_t hs) {
    const uint32_t warps = (a.H + hs - 1) / hs;
    const dim3 grid((a.T + qt - 1) / qt, a.nsplit), block(warps * 32);
    const size_t smem = win_attn_smem(a.H, a.D, a.RL, qt);
    if (hs == 1) {
        if (qt == 8) return launch<WinAttnArgs>(e, k_window_attn<VCH, 8, 1>, grid, block, smem, a);
        if (qt == 4) return launch<WinAttnArgs>(e, k_window_attn<VCH, 4, 1>, grid, block, smem, a);
        return launch<WinAttnArgs>(e, k_window_attn<VCH, 1, 1>, grid, block, smem, a);
    }
    if (qt == 4) return launch<WinAttnArgs>(e, k_window_attn<VCH, 4, 2>, grid, block, smem, a);
    return launch<WinAttnArgs>(e, k_window_attn<VCH, 1, 2>, grid, block, smem, a);
}
template <int VCH>
int win_attn_optin_v(int smem) {
    CK(cudaFuncSetAttribute((const void *)k_window_attn<VCH, 8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_window_attn<VCH, 4, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_window_attn<VCH, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_window_attn<VCH, 4, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_window_attn<VCH, 1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    return 0;
}
constexpr size_t kWinSmemMax = 200 * 1024;
// query tokens per block of a prefill portion: the largest of 8 / 4 / 1 whose shared memory fits (heads above 16: two per warp, 4 at most)
uint32_t win_attn_qt(const Layer &L) {
    const uint32_t hs = L.H > 16 ? 2u : 1u;
    for (uint32_t qt : {8u, 4u, 1u}) if (!(hs == 2 && qt == 8) && win_attn_smem(L.H, L.dim, L.RL, qt) <= kWinSmemMax) return qt;
    return 0;
}
int win_attn_launch(LayeredEngine *e, const Layer &L, const WinAttnArgs &a) {
    const uint32_t hs = L.H > 16 ? 2u : 1u, qt = a.T <= kGemvMaxM ? 1u : win_attn_qt(L);
    if (L.dim <= 32) return win_attn_launch_v<1>(e, a, qt, hs);
    if (L.dim <= 64) return win_attn_launch_v<2>(e, a, qt, hs);
    if (L.dim <= 128) return win_attn_launch_v<4>(e, a, qt, hs);
    return win_attn_launch_v<8>(e, a, qt, hs);
}

constexpr size_t kSelStageMax = 160 * 1024;      // dynamic shared memory the time-parallel scan may stage its inputs in (32 KB of maps are static)
template <int LG>
int sel_scan_optin() {
    CK(cudaFuncSetAttribute((const void *)k_selective_scan_par<LG, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSelStageMax));
    return 0;
}
template <int LG>
int sel_scan_launch(LayeredEngine *e, const SelScanArgs &a) {
    if (a.T > 32) {
        const dim3 grid(((size_t)a.C * LG + 31u) / 32u), block(32, a.T >= 256 ? 32 : 8);
        const size_t stage = sel_scan_stage_bytes(a.T, LG);
        if (stage <= kSelStageMax) return launch<SelScanArgs>(e, k_selective_scan_par<LG, true>, grid, block, stage, a);
        return launch<SelScanArgs>(e, k_selective_scan_par<LG, false>, grid, block, 0, a);
    }
    return launch<SelScanArgs>(e, k_selective_scan<LG>, dim3(((size_t)a.C * LG + 255u) / 256u), dim3(256), 0, a);
}

int conv_launch(LayeredEngine *e, const ConvArgs &ca) {
    int r;
    if ((r = launch<ConvArgs>(e, k_conv, dim3(ew_grid((size_t)ca.T * ca.C)), dim3(256), 0, ca))) return r;
    if (ca.K > 1 && (r = launch<ConvArgs>(e, k_conv_state, dim3((ca.C + 127) / 128), dim3(128), 0, ca))) return r;
    return 0;
}

// window attention and selective scan on the same input: one product gives [q | k | x | g | z]; q, k pass their convolution (tail in
// the slot), the convolved k is cached as value and key; x passes its convolution with bias and silu, gives [dt | B | C], dt its
// softplus; the two output products are summed with the layer's scales
int mix_window_ssm(LayeredEngine *e, const Layer &L, const Run &run, const Ctx &cx) {
    const uint32_t E = e->E, T = cx.T, H = L.H, G = L.G, D = L.dim, C = L.mC, N = L.mN, R = L.mR;
    const uint32_t QK = H * D + G * D, P = QK + C + H * D + C, g0 = QK + C, z0 = g0 + H * D;
    int r;
    const bool small = T <= kGemvMaxM;
    if (small) {      // both convolutions are epilogues of the product (a warp owns a channel and its tail)
        GemmArgs pj = plain(e->hm, E, L.proj, e->b_p, P, T, nullptr, EPI_CONV_RANGES);
        pj.cr[0] = {0, QK, L.a_conv, nullptr, cx.st + run.st_conv, e->b_qk, L.a_taps, 0};
        pj.cr[1] = {QK, QK + C, L.m_conv, L.m_conv_b, cx.st + run.st_conv2, e->b_xc, L.m_taps, 1};
        if ((r = gemm(e, pj, 1, T))) return r;
    } else if ((r = gemm(e, plain(e->hm, E, L.proj, e->b_p, P, T), 1, T))) return r;
    // the two sides share nothing after the product: the scan side runs on a second stream and joins before the residual update
    if (e->branch_streams) { CK(cudaEventRecord(e->ev_fork, e->stream)); e->cur = e->side; CK(cudaStreamWaitEvent(e->side, e->ev_fork, 0)); }
    // right
    if (!small && (r = conv_launch(e, ConvArgs{e->b_p + QK, P, L.m_conv, L.m_conv_b, cx.st + run.st_conv2, e->b_xc, T, C, L.m_taps, C, 1}))) return r;
    if ((r = gemm(e, plain(e->b_xc, C, L.xw, e->b_dbc, R + 2 * N, T), 1, T))) return r;
    if (!small && (r = gemm(e, plain(e->b_dbc, R + 2 * N, L.dtw, e->b_dt, C, T, L.dt_b, EPI_SOFTPLUS), 1, T))) return r;
    SelScanArgs sa{e->b_dt, e->b_xc, e->b_dbc, R + 2 * N, R, R + N, L.A, L.Dv, e->b_p + z0, P, cx.st + run.st_S, e->b_y, T, C, N,
                   small ? L.dt_wf : nullptr, L.dt_b, R, e->f32 ? 0u : 1u};
    if (N <= 4) r = sel_scan_launch<1>(e, sa);
    else if (N <= 8) r = sel_scan_launch<2>(e, sa);
    else if (N <= 16) r = sel_scan_launch<4>(e, sa);
    else if (N <= 32) r = sel_scan_launch<8>(e, sa);
    else if (N <= 64) r = sel_scan_launch<16>(e, sa);
    else r = sel_scan_launch<32>(e, sa);
    if (r) return r;
    GemmArgs ro = plain(e->b_y, C, L.mo, e->d2, E, T);
    ro.c_scale = L.right_scale; ro.c_mode = C_SCALE;
    if ((r = gemm(e, ro, 1, T))) return r;
    if (e->branch_streams) { CK(cudaEventRecord(e->ev_join, e->side)); e->cur = e->stream; }
    // left
    if (!small && (r = conv_launch(e, ConvArgs{e->b_p, P, L.a_conv, nullptr, cx.st + run.st_conv, e->b_qk, T, QK, L.a_taps, QK, 0}))) return r;
    QkPrepArgs qa{e->b_qk, QK, e->b_qk + H * D, QK, L.temp, L.scale, run.cache, cx.table, H, G, D, L.RL, cx.pos0, e->eps, cx.pos_ptr};
    if ((r = launch<QkPrepArgs>(e, k_qk_prepare, dim3(T), dim3(256), 0, qa))) return r;
    WinAttnArgs wa{e->b_qk, QK, run.cache, cx.table, e->b_p + g0, P, L.talk, L.slopes, e->b_a, T, H, G, D, L.RL, cx.pos0, L.window, L.softcap, cx.pos_ptr, 1u, e->b_wpart, e->b_wtick};
    if (small) {      // short portions: the key pages of the window are dealt out to several blocks (two pages each at least)
        const uint32_t reach = cx.pos_ptr ? e->max_tokens : cx.pos0 + T;      // a captured step does not know the position: the most pages a window can span
        const uint32_t pages = std::min(reach, L.window + T) / kPage + 1u;
        wa.nsplit = std::max(1u, std::min(kSplitMax, pages / 2u));
    }
    if ((r = win_attn_launch(e, L, wa))) return r;
    GemmArgs lo = plain(e->b_a, H * D, L.o, e->d, E, T);
    lo.c_scale = L.left_scale; lo.c_mode = C_SCALE;
    if ((r = gemm(e, lo, 1, T))) return r;
    if (e->branch_streams) CK(cudaStreamWaitEvent(e->stream, e->ev_join, 0));
    return 0;
}

// a sublayer's last product (into e->d); with the residual epilogue armed it updates e->x and writes the next sublayer's input instead
int last_product(LayeredEngine *e, GemmArgs g, uint32_t T) {
    if (e->res.on) {
        g.res_x = e->x; g.res_out = e->res.out; g.res_keep = e->res.keep;
        g.res_pw = e->res.post.w; g.res_pb = e->res.post.b; g.res_pa = e->res.post.alpha;
        g.res_nw = e->res.pre.w; g.res_nb = e->res.pre.b; g.res_na = e->res.pre.alpha;
    }
    return gemm(e, g, 1, T);
}

// ---- grouped-query differential attention ----
template <int VCH>
int diff_attn_launch_v(LayeredEngine *e, const DiffAttnArgs &a, uint32_t qt, uint32_t hpb, size_t smem) {
    const dim3 grid((a.T + qt - 1) / qt, a.nsplit, (a.H + hpb - 1) / hpb), block(hpb * 32);
    if (qt == 4) return launch<DiffAttnArgs>(e, k_diff_attn<VCH, 4>, grid, block, smem, a);
    return launch<DiffAttnArgs>(e, k_diff_attn<VCH, 1>, grid, block, smem, a);
}
template <int VCH>
int diff_attn_optin_v(int smem) {
    CK(cudaFuncSetAttribute((const void *)k_diff_attn<VCH, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    CK(cudaFuncSetAttribute((const void *)k_diff_attn<VCH, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    return 0;
}
inline int diff_vch(uint32_t vdim) { return vdim <= 32 ? 0 : vdim <= 64 ? 1 : vdim <= 128 ? 2 : 3; }

// one product gives [q | k | v] with their biases; q turns in place, the turned k and v go to the cache pages (this layer's, or none
// when it reads another layer's); both maps of a head in one warp; output product with its bias
int mix_diff_attn(LayeredEngine *e, const Layer &L, const Run &run, const Ctx &cx) {
    const uint32_t E = e->E, T = cx.T, H = L.H, G = L.G, D = L.dim, VD = L.vdim;
    const bool has_kv = L.kv_from < 0;
    const uint32_t QW = H * 2 * D, KW = G * 2 * D, P = QW + (has_kv ? KW + G * VD : 0);
    int r;
    if ((r = gemm(e, plain(e->hm, E, L.proj, e->b_p, P, T, L.proj_b), 1, T))) return r;
    if (has_kv || L.rot_tab) {
        RopeKvArgs ra{e->b_p, P, QW, QW + KW, has_kv ? 1u : 0u, run.cache, cx.table, T, H, G, 2u, D, VD, L.RL, L.rot_dims, cx.pos0, L.rot_tab, cx.pos_ptr};
        if ((r = launch<RopeKvArgs>(e, k_rope_kv, dim3(T), dim3(256), 0, ra))) return r;
    }
    const bool small = T <= kGemvMaxM;
    const uint32_t hpb = small ? L.a_hpb1 : L.a_hpb, ngk = small ? L.a_ngk1 : L.a_ngk;
    DiffAttnArgs aa{e->b_p, P, run.cache, cx.table, e->b_a, T, H, G, D, VD, L.RL, cx.pos0, L.scale, L.lambda, 1.0f - L.diff, e->eps, cx.pos_ptr, 1u, e->b_dpart, e->b_dtick, ngk};
    if (cx.pos_ptr) aa.nsplit = kSplitMax;           // the position is not known here: splits without keys write empty partials
    else if (small) aa.nsplit = std::max(1u, std::min(kSplitMax, (cx.pos0 + T + kPage - 1) / kPage / 2u));
    const uint32_t qt = small ? 1u : L.a_qt;
    const size_t smem = diff_attn_smem(D, VD, ngk, qt, hpb, diff_attn_vec(D, VD, P));
    switch (diff_vch(VD)) {
        case 0: r = diff_attn_launch_v<1>(e, aa, qt, hpb, smem); break;
        case 1: r = diff_attn_launch_v<2>(e, aa, qt, hpb, smem); break;
        case 2: r = diff_attn_launch_v<4>(e, aa, qt, hpb, smem); break;
        default: r = diff_attn_launch_v<8>(e, aa, qt, hpb, smem);
    }
    if (r) return r;
    return last_product(e, plain(e->b_a, H * VD, L.o, e->d, E, T, L.o_b), T);
}

// ---- state-space duality (Mamba-2) ----
// one product gives [z | x | B | C | dt]; [x | B | C] passes its convolution with bias and silu (tail in the slot; for short portions
// as the product's epilogue); the scan makes dt and the decay itself; gate, group norm and gain; output product
int mix_ssd(LayeredEngine *e, const Layer &L, const Run &run, const Ctx &cx) {
    const uint32_t E = e->E, T = cx.T, Hn = L.H, Pd = L.vdim, N = L.mN, G = L.G, inner = Hn * Pd, XW = inner + 2 * G * N, Pw = inner + XW + Hn;
    int r;
    const bool small = T <= kGemvMaxM;
    if (small) {
        GemmArgs pj = plain(e->hm, E, L.proj, e->b_p, Pw, T, nullptr, EPI_CONV_RANGES);
        pj.cr[0] = {inner, inner + XW, L.m_conv, L.m_conv_b, cx.st + run.st_conv, e->b_sdx, L.m_taps, 1};
        if ((r = gemm(e, pj, 1, T))) return r;
    } else if ((r = gemm(e, plain(e->hm, E, L.proj, e->b_p, Pw, T), 1, T)) ||
               (r = conv_launch(e, ConvArgs{e->b_p + inner, Pw, L.m_conv, L.m_conv_b, cx.st + run.st_conv, e->b_sdx, T, XW, L.m_taps, XW, 1}))) return r;
    SsdArgs sa{e->b_sdx, XW, e->b_p + inner + XW, Pw, L.dt_b, L.A, L.Dv, cx.st + run.st_S, e->b_sdy, T, Hn, Pd, N, G, 0u, 0u, e->b_sseg, e->b_p, Pw};
    const uint32_t nseg = T >= 64 ? std::min(kRetSegs, T / 32u) : 1u;
    if (nseg > 1) sa.seg_len = (T + nseg - 1u) / nseg;
    // columns per warp: four (fewest staged bytes per FMA) where the grid still gives every SM a dozen warps, else one
    const uint32_t cpw = (size_t)Hn * Pd / 4u * nseg >= (size_t)e->num_sms * 12u ? 4u : 1u;
    const dim3 grid((Pd + 8u * cpw - 1u) / (8u * cpw), Hn, nseg), block(256);
    for (uint32_t pass = (nseg > 1 ? 1u : 0u); pass <= (nseg > 1 ? 2u : 0u); pass++) {
        sa.mode = pass;
#define SSD_LAUNCH(DCH) (cpw == 4 ? launch<SsdArgs>(e, k_ssd_scan<DCH, 4>, grid, block, 0, sa) : launch<SsdArgs>(e, k_ssd_scan<DCH, 1>, grid, block, 0, sa))
        if (N <= 32) r = SSD_LAUNCH(1);
        else if (N <= 64) r = SSD_LAUNCH(2);
        else if (N <= 128) r = SSD_LAUNCH(4);
        else r = SSD_LAUNCH(8);
#undef SSD_LAUNCH
        if (r) return r;
        if (pass == 1) {
            SsdChainArgs ca{cx.st + run.st_S, e->b_sseg, e->b_p + inner + XW, Pw, L.dt_b, L.A, Hn, Pd, N, T, sa.seg_len, nseg};
            if ((r = launch<SsdChainArgs>(e, k_ssd_chain, dim3(std::min(8u, (Pd * N + 255u) / 256u), Hn), dim3(256), 0, ca))) return r;
        }
    }
    // the scan's output leaves gated; its norm in equal parts is the prologue of the output product for short portions (where the
    // parts are multiples of 8 columns), a kernel of its own otherwise
    const uint32_t plen = inner / L.parts;
    if (small && (L.parts == 1 || (L.parts <= 32 && plen % 8u == 0))) {
        GemmArgs o = plain(e->b_sdy, inner, L.o, e->d, E, T);
        o.a_norm_w = L.gn; o.a_eps = e->eps; o.a_parts = L.parts;
        if (L.parts == 1) o.a_parts = 0;          // one part: the plain instance's whole-row norm
        return last_product(e, o, T);
    }
    GroupNormArgs oa{e->b_sdy, L.gn, e->b_a, T, inner, L.parts, e->eps};
    if ((r = launch<GroupNormArgs>(e, k_group_norm, dim3(T * L.parts), dim3(small ? 1024 : 128), 0, oa))) return r;
    return last_product(e, plain(e->b_a, inner, L.o, e->d, E, T), T);
}

int mix(LayeredEngine *e, const Layer &L, const Run &run, const Ctx &cx) {
    switch (L.type) {
        case MIX_RGLRU: return mix_rglru(e, L, run, cx);
        case MIX_LATENT_ATTN: return mix_latent_attn(e, L, run, cx);
        case MIX_RETENTION: return mix_retention(e, L, run, cx);
        case MIX_DIFF_ATTN: return mix_diff_attn(e, L, run, cx);
        case MIX_SSD: return mix_ssd(e, L, run, cx);
        default: return mix_window_ssm(e, L, run, cx);
    }
}

// dense feed-forward with the PolyNorm activation: e->h2 -> e->d
int ff_dense(LayeredEngine *e, const Layer &L, uint32_t T) {
    int r;
    if ((r = gemm(e, plain(e->h2, e->E, L.up, e->b_f, L.ff, T), 1, T))) return r;
    if (T <= kGemvMaxM) {      // short portions: the activation is the prologue of the second product
        GemmArgs dn = plain(e->b_f, L.ff, L.down, e->d, e->E, T);
        dn.a_poly = L.act; dn.a_eps = e->eps;
        return gemm(e, dn, 1, T);
    }
    PolyArgs pa{e->b_f, L.ff, L.act, T, L.ff, e->eps};
    if ((r = launch<PolyArgs>(e, k_polynorm, dim3(T), dim3(256), 0, pa))) return r;
    return gemm(e, plain(e->b_f, L.ff, L.down, e->d, e->E, T), 1, T);
}

// gated dense feed-forward: e->h2 -> e->d.  Short portions: gate and up rows meet in the matrix-vector kernel; long ones pass k_glu
int ff_glu_dense(LayeredEngine *e, const Layer &L, uint32_t T) {
    int r;
    if (T <= kGemvMaxM) {
        GemmArgs u = plain(e->h2, e->E, L.up, e->b_f2, L.ff, T);
        u.N = L.ff; u.glu = 1u;
        if ((r = gemm(e, u, 1, T))) return r;
    } else {
        if ((r = gemm(e, plain(e->h2, e->E, L.up, e->b_f, 2 * L.ff, T), 1, T))) return r;
        GluArgs ga{e->b_f, 2 * L.ff, e->b_f2, L.ff, nullptr, T, L.ff, 0u};
        if ((r = launch<GluArgs>(e, k_glu, dim3(ew_grid((size_t)T * L.ff)), dim3(256), 0, ga))) return r;
    }
    return last_product(e, plain(e->b_f2, L.ff, L.down, e->d, e->E, T), T);
}

// experts chosen by sigmoid scores: e->h2 -> the rows of e->b_eo (one per token and choice, in expert order) and, with a shared expert,
// e->b_so and the gate logits e->b_sg; the residual kernel adds them up.  The score weights the expert's INPUT; the experts have no
// bias, so act(s g) (s u) of the unweighted products g, u is the same number.  The shared expert runs on a second stream.
int ff_moe_scored(LayeredEngine *e, const Layer &L, uint32_t T) {
    const uint32_t E = e->E, NL = L.NE + (L.sh_gate ? 1u : 0u);
    const bool small = T <= kGemvMaxM;
    int r;
    if (L.has_shared && e->branch_streams) CK(cudaEventRecord(e->ev_fork, e->stream));
    float *wrow = L.score_in ? e->b_wrow : nullptr;
    RouteArgs ra{e->h2, L.router, e->b_idx, e->b_wt, e->b_cnt, e->b_off, e->b_fill, e->b_slot, e->b_rows, T, L.NE, L.top, E, L.route_mode, L.sh_gate ? 1u : 0u, e->b_sg, wrow};
    if (small) { if ((r = launch<RouteArgs>(e, k_route_small, dim3(1), dim3(1024), route_smem(NL, 1024), ra))) return r; }
    else if ((r = launch<RouteArgs>(e, k_route, dim3(T), dim3(256), route_smem(NL, 256), ra)) || (r = launch<RouteArgs>(e, k_route_place, dim3(1), dim3(1024), 0, ra))) return r;
    GemmArgs u{};
    u.A = e->h2; u.lda = E; u.W = L.up.p; u.ldw = E; u.M = T; u.K = E; u.a_gmod = 1;
    u.g_off = e->b_off; u.a_rows = e->b_rows; u.w_gstride = (uint64_t)2 * L.ff * E;
    if (small) { u.C = e->b_hb; u.ldc = L.ff; u.N = L.ff; u.glu = L.glu_kind; u.glu_limit = L.limit; u.row_scale = wrow; }
    else { u.C = e->b_hg; u.ldc = 2 * L.ff; u.N = 2 * L.ff; }
    if ((r = gemm(e, u, L.NE, T, false, T * L.top))) return r;
    if (!small) {
        GluArgs ga{e->b_hg, 2 * L.ff, e->b_hb, L.ff, wrow, T * L.top, L.ff, L.glu_kind == 3u ? 2u : 1u, L.limit};
        if ((r = launch<GluArgs>(e, k_glu, dim3(ew_grid((size_t)T * L.top * L.ff)), dim3(256), 0, ga))) return r;
    }
    GemmArgs dn{};
    dn.A = e->b_hb; dn.lda = L.ff; dn.W = L.down.p; dn.ldw = L.ff; dn.C = e->b_eo; dn.ldc = E; dn.M = T; dn.N = E; dn.K = L.ff; dn.a_gmod = 1;
    dn.g_off = e->b_off; dn.w_gstride = (uint64_t)E * L.ff;
    if ((r = gemm(e, dn, L.NE, T, false, T * L.top))) return r;
    if (!L.has_shared) return 0;
    if (e->branch_streams) { e->cur = e->side; CK(cudaStreamWaitEvent(e->side, e->ev_fork, 0)); }
    if (small) {
        GemmArgs su = plain(e->h2, E, L.sup, e->b_sh2, L.sff, T);
        su.N = L.sff; su.glu = L.glu_kind; su.glu_limit = L.slimit;
        if ((r = gemm(e, su, 1, T))) return r;
    } else {
        if ((r = gemm(e, plain(e->h2, E, L.sup, e->b_sh, 2 * L.sff, T), 1, T))) return r;
        GluArgs ga{e->b_sh, 2 * L.sff, e->b_sh2, L.sff, nullptr, T, L.sff, L.glu_kind == 3u ? 2u : 1u, L.slimit};
        if ((r = launch<GluArgs>(e, k_glu, dim3(ew_grid((size_t)T * L.sff)), dim3(256), 0, ga))) return r;
    }
    if ((r = gemm(e, plain(e->b_sh2, L.sff, L.sdown, e->b_so, E, T), 1, T))) return r;
    if (e->branch_streams) { CK(cudaEventRecord(e->ev_join, e->side)); e->cur = e->stream; CK(cudaStreamWaitEvent(e->stream, e->ev_join, 0)); }
    return 0;
}

// x += dyt_post(sublayer output); out = dyt_pre(x) when a sublayer follows.  moe: the output is the experts' rows (+ the gated shared expert)
int dyt_residual(LayeredEngine *e, const Layer *moe, const Dyt &post, const Dyt *pre, float *out, float *keep, uint32_t T) {
    DytResArgs a{e->x, moe ? nullptr : e->d, moe ? e->b_eo : nullptr, e->b_slot, moe ? moe->top : 0u, moe && moe->has_shared ? e->b_so : nullptr, e->b_sg,
                 post, pre ? *pre : Dyt{}, pre ? out : nullptr, keep, T, e->E};
    return launch<DytResArgs>(e, k_dyt_residual, dim3(ew_grid((size_t)T * e->E)), dim3(256), 0, a);
}

// dense feed-forward with the exact gelu as the first product's epilogue: e->h2 -> e->d
int ff_dense_gelu(LayeredEngine *e, const Layer &L, uint32_t T) {
    int r;
    if ((r = gemm(e, plain(e->h2, e->E, L.up, e->b_f, L.ff, T, nullptr, EPI_GELU_ERF), 1, T))) return r;
    return gemm(e, plain(e->b_f, L.ff, L.down, e->d, e->E, T), 1, T);
}

// hyper-connected residual streams: the update after a sublayer (hc, ls: its connection weights and layer scale; moe: its output is the
// chosen experts' rows) and the input norm of the sublayer that follows (next_hc's `in` weights, gain next_w, into out); with tokens
// the streams are filled from the embedding instead
int hc_step(LayeredEngine *e, const float *hc, const float *ls, const Layer *moe, const float *next_hc, const float *next_w, float *out, float *keep, uint32_t T,
            const uint32_t *tok_dev = nullptr, const uint32_t *pos_ptr = nullptr) {
    HcArgs a{};
    a.xs = e->xs; a.s_stride = (size_t)e->chunk_cap * e->E; a.S = e->S;
    if (!tok_dev) {
        if (moe) { a.eo = e->b_eo; a.slot = e->b_slot; a.wt = e->b_wt; a.top = moe->top; a.shared = moe->has_shared ? e->b_so : nullptr; }
        else a.y = e->d;
    }
    a.ls = ls; a.hc = hc; a.mult = e->res_mult;
    a.next_in = next_hc; a.next_w = next_w; a.out = next_hc ? out : nullptr; a.keep = keep;
    a.T = T; a.E = e->E; a.eps = e->eps;
    a.tokens = tok_dev; a.pos_ptr = pos_ptr; a.embed = e->embed.p; a.emb_scale = e->emb_scale;
    // a short portion is a few lone blocks: wide ones, so that a thread's chain of loads stays short
    const dim3 block(T <= kGemvMaxM && e->E >= 2048 ? 1024 : (T <= kGemvMaxM && e->E >= 1024 ? 512 : 256));
#define HC_LAUNCH(SC) (e->f32 ? launch<HcArgs>(e, k_hc_step<float, SC>, dim3(T), block, 0, a) : launch<HcArgs>(e, k_hc_step<__nv_bfloat16, SC>, dim3(T), block, 0, a))
    if (e->S <= 1) return HC_LAUNCH(1);
    if (e->S <= 2) return HC_LAUNCH(2);
    if (e->S <= 4) return HC_LAUNCH(4);
    return HC_LAUNCH((int)kMaxStreams);
#undef HC_LAUNCH
}

int sandwich(LayeredEngine *e, const float *d, const float *w_post, const float *w_pre, float *out, float *keep, uint32_t T, const float *d2 = nullptr) {
    SandwichArgs a{e->x, d, w_post, w_pre, out, keep, T, e->E, e->eps, d2};
    // a short portion is a few lone blocks: wide ones, so that a thread's chain of loads stays short
    return launch<SandwichArgs>(e, k_sandwich, dim3(T), dim3(T <= kGemvMaxM && e->E >= 2048 ? 1024 : (T <= kGemvMaxM && e->E >= 1024 ? 512 : 256)), 0, a);
}

// every layer run over T tokens (x already holds their embeddings) of the sequence in `slot`, whose first token sits at pos0
// (+ *pos_ptr: a captured decode step keeps the position on the device and uses a fixed number of key splits)
int run_layers(LayeredEngine *e, uint32_t slot, uint32_t T, uint32_t pos0, const uint32_t *pos_ptr = nullptr) {
    const uint32_t E = e->E;
    float *st = e->state + (size_t)slot * e->slot_floats;
    const Ctx cx{st, e->table + (size_t)slot * e->n_pages, T, pos0, pos_ptr};
    int r;
    e->cur = e->stream;
    for (size_t ri = 0; ri < e->runs.size(); ri++) {
        const Run &run = e->runs[ri];
        const Layer &L = e->layers[run.layer];
        float *keep = e->keep ? e->keep + ri * (size_t)e->chunk_cap * E : nullptr;
        if (e->form == FORM_HYPER) {
            // e->hm already holds the mixer's input (from the embedding step or the update before); every update also prepares the
            // input of the sublayer that follows (this layer's feed-forward, or the next run's mixer)
            const Layer *NX = ri + 1 < e->runs.size() ? &e->layers[e->runs[ri + 1].layer] : nullptr;
            if ((r = mix(e, L, run, cx))) return r;
            if (!L.has_mlp) { if ((r = hc_step(e, L.hc1, L.ls1, nullptr, NX ? NX->hc1 : nullptr, NX ? NX->ln1 : nullptr, e->hm, keep, T))) return r; continue; }
            if ((r = hc_step(e, L.hc1, L.ls1, nullptr, L.hc2, L.ln2, e->h2, nullptr, T))) return r;
            const bool moe = L.ff_kind == FF_MOE_SCORED;
            if ((r = moe ? ff_moe_scored(e, L, T) : ff_dense_gelu(e, L, T))) return r;
            if ((r = hc_step(e, L.hc2, L.ls2, moe ? &L : nullptr, NX ? NX->hc1 : nullptr, NX ? NX->ln1 : nullptr, e->hm, keep, T))) return r;
            continue;
        }
        if (e->form == FORM_SANDWICH && e->norm_kind == NORM_DYT) {
            // the same two updates through Dynamic-Tanh norms; e->hm already holds norm1(x) (from the embedding or the update before)
            const Dyt *next_d1 = ri + 1 < e->runs.size() ? &e->layers[e->runs[ri + 1].layer].d1 : nullptr;
            // short portions: a residual update is the epilogue of the product before it (the norms are elementwise), except after routed experts
            const bool ride = T <= kGemvMaxM;
            const Dyt *after_mix = L.has_mlp ? &L.d2 : next_d1;
            e->res.on = ride; e->res.post = L.d1b; e->res.pre = after_mix ? *after_mix : Dyt{};
            e->res.out = after_mix ? (L.has_mlp ? e->h2 : e->hm) : nullptr; e->res.keep = L.has_mlp ? nullptr : keep;
            r = mix(e, L, run, cx);
            e->res.on = false;
            if (r) return r;
            if (!ride && (r = dyt_residual(e, nullptr, L.d1b, after_mix, L.has_mlp ? e->h2 : e->hm, L.has_mlp ? nullptr : keep, T))) return r;
            if (L.has_mlp && L.ff_kind == FF_MOE_SCORED) {
                if ((r = ff_moe_scored(e, L, T)) || (r = dyt_residual(e, &L, L.d2b, next_d1, e->hm, keep, T))) return r;
            } else if (L.has_mlp) {
                e->res.on = ride; e->res.post = L.d2b; e->res.pre = next_d1 ? *next_d1 : Dyt{}; e->res.out = next_d1 ? e->hm : nullptr; e->res.keep = keep;
                r = ff_glu_dense(e, L, T);
                e->res.on = false;
                if (r) return r;
                if (!ride && (r = dyt_residual(e, nullptr, L.d2b, next_d1, e->hm, keep, T))) return r;
            }
            continue;
        }
        if (e->form == FORM_SANDWICH) {
            // x <- x + norm1b(mixer(norm1 x)), x <- x + norm2b(ff(norm2 x)): each residual update also norms the updated x for the
            // sublayer that follows (this layer's feed-forward, or the next run's mixer)
            const float *next_n1 = ri + 1 < e->runs.size() ? e->layers[e->runs[ri + 1].layer].n1 : nullptr;
            if (ri == 0 && (r = sandwich(e, nullptr, nullptr, L.n1, e->hm, nullptr, T))) return r;
            if ((r = mix(e, L, run, cx))) return r;
            const float *d2 = L.type == MIX_WINDOW_SSM ? e->d2 : nullptr;      // the scan side of a two-sided mixer
            if (L.has_mlp) {
                if ((r = sandwich(e, e->d, L.n1b, L.n2, e->h2, nullptr, T, d2)) || (r = ff_dense(e, L, T)) ||
                    (r = sandwich(e, e->d, L.n2b, next_n1, next_n1 ? e->hm : nullptr, keep, T))) return r;
            } else if ((r = sandwich(e, e->d, L.n1b, next_n1, next_n1 ? e->hm : nullptr, keep, T, d2))) return r;
            continue;
        }
        if (run.add_embed) { k_add<<<ew_grid((size_t)T * E), 256, 0, e->stream>>>(e->x, e->x0, (size_t)T * E); CK(cudaGetLastError()); e->launches++; }
        {
            NormShiftArgs a{e->x, L.norm1, L.has_mlp ? L.norm2 : nullptr, L.shift, st + run.st_prev, e->hm, L.has_mlp ? e->h2 : nullptr, T, E, e->eps};
            if ((r = launch<NormShiftArgs>(e, k_norm_shift, dim3(T > 1 ? T - 1 : 1), dim3(256), 0, a))) return r;
            if (L.has_mlp && e->branch_streams) CK(cudaEventRecord(e->ev_fork, e->stream));
        }
        if ((r = mix(e, L, run, cx))) return r;
        CombineArgs c{e->x, e->d, nullptr, nullptr, nullptr, nullptr, keep, T, E, 0};
        if (L.has_mlp) {
            // The layer is parallel: the feed-forward reads h2 = norm2(x) of the SAME x and shares no buffer with the mixer, so its
            // kernels go to a second stream (a parallel branch of the captured decode graph) and join before the residual update.
            if (e->branch_streams) { e->cur = e->side; CK(cudaStreamWaitEvent(e->side, e->ev_fork, 0)); }
            RouteArgs ra{e->h2, L.router, e->b_idx, e->b_wt, e->b_cnt, e->b_off, e->b_fill, e->b_slot, e->b_rows, T, L.NE, L.top, E};
            if (T <= kGemvMaxM) { if ((r = launch<RouteArgs>(e, k_route_small, dim3(1), dim3(1024), route_smem(L.NE, 1024), ra))) return r; }
            else if ((r = launch<RouteArgs>(e, k_route, dim3(T), dim3(256), route_smem(L.NE, 256), ra)) ||
                     (r = launch<RouteArgs>(e, k_route_place, dim3(1), dim3(1024), 0, ra))) return r;
            GemmArgs u{};
            u.A = e->h2; u.lda = E; u.W = L.up.p; u.ldw = E; u.C = e->b_hb; u.ldc = L.ff; u.M = T; u.N = L.ff; u.K = E; u.a_gmod = 1;
            u.g_off = e->b_off; u.a_rows = e->b_rows; u.w_gstride = (uint64_t)L.ff * E; u.epi = EPI_RELU2;
            if ((r = gemm(e, u, L.NE, T, false, T * L.top))) return r;
            GemmArgs dn{};
            dn.A = e->b_hb; dn.lda = L.ff; dn.W = L.down.p; dn.ldw = L.ff; dn.C = e->b_eo; dn.ldc = E; dn.M = T; dn.N = E; dn.K = L.ff; dn.a_gmod = 1;
            dn.g_off = e->b_off; dn.w_gstride = (uint64_t)E * L.ff;
            if ((r = gemm(e, dn, L.NE, T, false, T * L.top))) return r;
            if (L.has_shared) {      // a third branch: the shared expert depends on h2 only
                if (e->branch_streams) { e->cur = e->side2; CK(cudaStreamWaitEvent(e->side2, e->ev_fork, 0)); }
                if ((r = gemm(e, plain(e->h2, E, L.sup, e->b_sh, L.sff, T, nullptr, EPI_RELU2), 1, T)) || (r = gemm(e, plain(e->b_sh, L.sff, L.sdown, e->b_so, E, T), 1, T))) return r;
                if (e->branch_streams) { CK(cudaEventRecord(e->ev_join2, e->side2)); CK(cudaStreamWaitEvent(e->stream, e->ev_join2, 0)); }
            }
            c.eo = e->b_eo; c.slot = e->b_slot; c.wt = e->b_wt; c.shared = L.has_shared ? e->b_so : nullptr; c.top = L.top;
            e->cur = e->stream;
            if (e->branch_streams) { CK(cudaEventRecord(e->ev_join, e->side)); CK(cudaStreamWaitEvent(e->stream, e->ev_join, 0)); }
        }
        if ((r = launch<CombineArgs>(e, k_combine, dim3(ew_grid((size_t)T * E)), dim3(256), 0, c))) return r;
    }
    e->last_T = T;
    return 0;
}

int embed_tokens(LayeredEngine *e, uint32_t slot, const uint32_t *tok_dev, uint32_t T, const uint32_t *pos_ptr = nullptr, uint32_t pos0 = 0) {
    if (e->form == FORM_HYPER) {      // token row x scale into every stream, and the first sublayer's input norm
        e->cur = e->stream;
        const Layer &L0 = e->layers[e->runs[0].layer];
        return hc_step(e, nullptr, nullptr, nullptr, L0.hc1, L0.ln1, e->hm, nullptr, T, tok_dev, pos_ptr);
    }
    if (e->norm_kind == NORM_DYT) {      // token row x scale + pair row, the stack's input norm, and the first sublayer's input norm
        e->cur = e->stream;
        EmbedPairArgs a{tok_dev, pos_ptr, e->embed.p, e->pairs.p, e->x, e->hm, reinterpret_cast<uint32_t *>(e->state + (size_t)slot * e->slot_floats + e->st_tok),
                        T, e->E, e->buckets, e->mul_prev, e->mul_cur, e->emb_scale, e->embed_norm, e->layers[e->runs[0].layer].d1};
        const dim3 block(T <= kGemvMaxM && e->E >= 2048 ? 512 : (T <= kGemvMaxM && e->E >= 1024 ? 256 : 128));
        return e->f32 ? launch<EmbedPairArgs>(e, k_embed_pair<float>, dim3(T), block, 0, a) : launch<EmbedPairArgs>(e, k_embed_pair<__nv_bfloat16>, dim3(T), block, 0, a);
    }
    if (e->max_pos) {      // a learned position row joins the token row
        if (e->f32) k_embed_pos<float><<<T, 128, 0, e->stream>>>(tok_dev, pos_ptr, (const float *)e->embed.p, (const float *)e->pos_table.p, e->x, e->E, pos0);
        else k_embed_pos<__nv_bfloat16><<<T, 128, 0, e->stream>>>(tok_dev, pos_ptr, (const __nv_bfloat16 *)e->embed.p, (const __nv_bfloat16 *)e->pos_table.p, e->x, e->E, pos0);
        CK(cudaGetLastError());
        e->launches++;
        return 0;
    }
    if (e->f32) k_embed<float><<<T, 128, 0, e->stream>>>(tok_dev, pos_ptr, (const float *)e->embed.p, e->x, e->keep_x0 ? e->x0 : nullptr, e->E);
    else k_embed<__nv_bfloat16><<<T, 128, 0, e->stream>>>(tok_dev, pos_ptr, (const __nv_bfloat16 *)e->embed.p, e->x, e->keep_x0 ? e->x0 : nullptr, e->E);
    CK(cudaGetLastError());
    e->launches++;
    return 0;
}

// logits of `nw` rows of the current chunk (want_dev holds their indices) -> e->logits [nw][V]
int head_rows(LayeredEngine *e, uint32_t nw, const uint32_t *want_dev = nullptr) {
    if (e->form == FORM_HYPER) {
        k_final_ln<<<nw, nw <= kGemvMaxM && e->E >= 1024 ? 1024 : 256, 0, e->stream>>>(e->xs, (size_t)e->chunk_cap * e->E, e->S, want_dev ? want_dev : e->want_dev, e->final_norm, e->b_xn, e->E, e->eps);
        CK(cudaGetLastError());
        e->launches++;
        return gemm(e, plain(e->b_xn, e->E, e->head, e->logits, e->V, nw), 1, nw);
    }
    if (e->norm_kind == NORM_DYT) {
        k_final_dyt<<<nw, 256, 0, e->stream>>>(e->x, want_dev ? want_dev : e->want_dev, e->final_dyt, e->b_xn, e->E);
        CK(cudaGetLastError());
        e->launches++;
        return gemm(e, plain(e->b_xn, e->E, e->head, e->logits, e->V, nw), 1, nw);
    }
    k_final_norm<<<nw, 256, 0, e->stream>>>(e->x, want_dev ? want_dev : e->want_dev, e->final_norm, e->b_xn, e->E, e->eps, e->form == FORM_SANDWICH ? 1u : 0u);
    CK(cudaGetLastError());
    e->launches++;
    return gemm(e, plain(e->b_xn, e->E, e->head, e->logits, e->V, nw), 1, nw);
}

// One decode step of `slot`: the token ids_dev[*dpos] at position *dpos, logits of it in e->logits[0..V).  The position lives in
// the device word dpos, so the launch sequence is the same for every step: it is captured once per slot into a CUDA graph and
// replayed (NB200_FLAG_NO_GRAPH: launched directly).  The caller has reserved the page and set *dpos.
int decode_launches(LayeredEngine *e, uint32_t slot) {
    int r;
    if ((r = embed_tokens(e, slot, e->ids_dev, 1, e->dpos)) || (r = run_layers(e, slot, 1, 0, e->dpos))) return r;
    return head_rows(e, 1, e->zero_dev);
}

int decode_step(LayeredEngine *e, uint32_t slot) {
    if (!e->use_graph || e->keep) return decode_launches(e, slot);
    if (!e->graphs[slot]) {
        cudaGraph_t g = nullptr;
        const uint64_t before = e->launches;
        CK(cudaStreamBeginCapture(e->stream, cudaStreamCaptureModeThreadLocal));
        int r = decode_launches(e, slot);
        cudaError_t ce = cudaStreamEndCapture(e->stream, &g);
        e->graph_launches = (uint32_t)(e->launches - before);
        e->launches = before;
        if (r) { if (g) cudaGraphDestroy(g); return r; }
        if (ce != cudaSuccess) return fail(NB200_ECUDA, "graph capture failed: %s", cudaGetErrorString(ce));
        ce = cudaGraphInstantiate(&e->graphs[slot], g, 0);
        cudaGraphDestroy(g);
        if (ce != cudaSuccess) { e->graphs[slot] = nullptr; return fail(NB200_ECUDA, "graph instantiate failed: %s", cudaGetErrorString(ce)); }
    }
    CK(cudaGraphLaunch(e->graphs[slot], e->stream));
    e->launches += e->graph_launches;
    e->last_T = 1;
    return 0;
}

// ---------------- state manager ----------------
int seq_check(LayeredEngine *e, uint32_t seq) {
    if (seq >= e->seqs.size() || !e->seqs[seq].live) return fail(NB200_EINVAL, "sequence %u is not open", seq);
    return 0;
}

int reserve_pages(LayeredEngine *e, uint32_t seq, uint32_t tokens) {
    Seq &s = e->seqs[seq];
    const size_t have = s.pages.size(), need = (tokens + kPage - 1) / kPage;
    if (e->max_pos && tokens > e->max_pos) return fail(NB200_EINVAL, "sequence %u would reach %u tokens; the model has %u positions", seq, tokens, e->max_pos);
    if (need <= have) return 0;
    if (need - have > e->free_pages.size()) return fail(NB200_ENOMEM, "the cache is full: %u tokens asked for sequence %u, %zu pages free", tokens, seq, e->free_pages.size());
    for (size_t i = have; i < need; i++) { s.pages.push_back(e->free_pages.back()); e->free_pages.pop_back(); }
    CK(cudaMemcpyAsync(e->table + (size_t)seq * e->n_pages + have, s.pages.data() + have, (need - have) * 4, cudaMemcpyHostToDevice, e->stream));
    CK(cudaStreamSynchronize(e->stream));      // the source is pageable host memory owned by the vector
    return 0;
}

int lm_seq_open(nb200_engine *h, uint32_t *seq) {
    LayeredEngine *e = self(h);
    if (!seq) return fail(NB200_EINVAL, "null argument");
    CK(cudaSetDevice(e->device));
    for (uint32_t i = 0; i < e->seqs.size(); i++) {
        if (e->seqs[i].live) continue;
        e->seqs[i].live = true; e->seqs[i].len = 0; e->seqs[i].pages.clear();
        CK(cudaMemsetAsync(e->state + (size_t)i * e->slot_floats, 0, e->slot_floats * 4, e->stream));
        *seq = i;
        return 0;
    }
    return fail(NB200_ENOMEM, "all %u sequence slots are in use", e->max_seqs);
}

int lm_seq_close(nb200_engine *h, uint32_t seq) {
    LayeredEngine *e = self(h);
    int r;
    if ((r = seq_check(e, seq))) return r;
    Seq &s = e->seqs[seq];
    for (size_t i = s.pages.size(); i > 0; i--) e->free_pages.push_back(s.pages[i - 1]);
    s.pages.clear(); s.live = false; s.len = 0;
    if ((int)seq == e->gen_seq) e->gen_seq = -1;
    return 0;
}

// ---------------- step ----------------
// tokens already on the device at tok_dev[0..n); want (host, ascending, may be null) -> logits_host [n_want][V]
int step_dev(LayeredEngine *e, uint32_t seq, const uint32_t *tok_dev, uint32_t n, const uint32_t *want, uint32_t n_want, float *logits_host) {
    int r;
    Seq &s = e->seqs[seq];
    if ((r = reserve_pages(e, seq, s.len + n))) return r;
    uint32_t wi = 0;
    for (uint32_t c0 = 0; c0 < n; c0 += e->chunk_cap) {
        const uint32_t T = std::min(e->chunk_cap, n - c0);
        if ((r = embed_tokens(e, seq, tok_dev + c0, T, nullptr, s.len)) || (r = run_layers(e, seq, T, s.len))) return r;
        s.len += T;
        while (wi < n_want && want[wi] < c0 + T) {
            uint32_t idx[kWantBatch], nw = 0;
            while (nw < kWantBatch && wi + nw < n_want && want[wi + nw] < c0 + T) { idx[nw] = want[wi + nw] - c0; nw++; }
            CK(cudaMemcpyAsync(e->want_dev, idx, nw * 4, cudaMemcpyHostToDevice, e->stream));
            CK(cudaStreamSynchronize(e->stream));
            if ((r = head_rows(e, nw))) return r;
            CK(cudaMemcpyAsync(logits_host + (size_t)wi * e->V, e->logits, (size_t)nw * e->V * 4, cudaMemcpyDeviceToHost, e->stream));
            CK(cudaStreamSynchronize(e->stream));
            wi += nw;
        }
    }
    return 0;
}

int check_tokens(LayeredEngine *e, const uint32_t *tokens, uint32_t n) {
    for (uint32_t i = 0; i < n; i++) if (tokens[i] >= e->V) return fail(NB200_EINVAL, "token id %u outside the vocabulary of %u", tokens[i], e->V);
    return 0;
}

int lm_step(nb200_engine *h, uint32_t seq, const uint32_t *tokens, uint32_t n, const uint32_t *want, uint32_t n_want, float *logits) {
    LayeredEngine *e = self(h);
    int r;
    if (!tokens || n == 0 || (n_want && (!want || !logits))) return fail(NB200_EINVAL, "bad arguments");
    if ((r = seq_check(e, seq)) || (r = check_tokens(e, tokens, n))) return r;
    for (uint32_t i = 0; i < n_want; i++) if (want[i] >= n || (i && want[i] <= want[i - 1])) return fail(NB200_EINVAL, "want[] must be ascending indices into this step's tokens");
    CK(cudaSetDevice(e->device));
    if (n == 1) {          // a single token: the captured decode step
        Seq &s = e->seqs[seq];
        if ((r = reserve_pages(e, seq, s.len + 1))) return r;
        CK(cudaMemcpyAsync(e->ids_dev + s.len, tokens, 4, cudaMemcpyHostToDevice, e->stream));
        CK(cudaMemcpyAsync(e->dpos, &s.len, 4, cudaMemcpyHostToDevice, e->stream));
        if ((r = decode_step(e, seq))) return r;
        s.len += 1;
        if (n_want) CK(cudaMemcpyAsync(logits, e->logits, (size_t)e->V * 4, cudaMemcpyDeviceToHost, e->stream));
        CK(cudaStreamSynchronize(e->stream));
        return 0;
    }
    std::vector<uint32_t> done;
    for (uint32_t c0 = 0; c0 < n; c0 += e->max_tokens) {          // the staging buffer holds max_tokens ids
        const uint32_t m = std::min(e->max_tokens, n - c0);
        CK(cudaMemcpyAsync(e->ids_dev, tokens + c0, (size_t)m * 4, cudaMemcpyHostToDevice, e->stream));
        CK(cudaStreamSynchronize(e->stream));
        uint32_t w0 = 0, w1 = 0;
        while (w0 < n_want && want[w0] < c0) w0++;
        w1 = w0;
        done.clear();
        while (w1 < n_want && want[w1] < c0 + m) done.push_back(want[w1++] - c0);
        if ((r = step_dev(e, seq, e->ids_dev, m, done.data(), (uint32_t)done.size(), logits ? logits + (size_t)w0 * e->V : nullptr))) return r;
    }
    CK(cudaStreamSynchronize(e->stream));
    return 0;
}

int lm_step_timed(nb200_engine *h, uint32_t seq, const uint32_t *tokens, uint32_t n, uint32_t reps, float *ms) {
    LayeredEngine *e = self(h);
    int r;
    if (!tokens || !n || !reps || !ms || n > e->max_tokens) return fail(NB200_EINVAL, "bad arguments");
    if ((r = seq_check(e, seq)) || (r = check_tokens(e, tokens, n))) return r;
    CK(cudaSetDevice(e->device));
    float *slot = e->state + (size_t)seq * e->slot_floats;
    const uint32_t len0 = e->seqs[seq].len;
    CK(cudaMemcpyAsync(e->ids_dev, tokens, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
    CK(cudaMemcpyAsync(e->state_bak, slot, e->slot_floats * 4, cudaMemcpyDeviceToDevice, e->stream));
    cudaEvent_t ev[2];
    CK(cudaEventCreate(&ev[0])); CK(cudaEventCreate(&ev[1]));
    float total = 0.0f;
    for (uint32_t rep = 0; rep <= reps; rep++) {           // rep 0 is the untimed run
        CK(cudaMemcpyAsync(slot, e->state_bak, e->slot_floats * 4, cudaMemcpyDeviceToDevice, e->stream));
        e->seqs[seq].len = len0;
        CK(cudaEventRecord(ev[0], e->stream));
        if ((r = step_dev(e, seq, e->ids_dev, n, nullptr, 0, nullptr))) break;
        CK(cudaEventRecord(ev[1], e->stream));
        CK(cudaStreamSynchronize(e->stream));
        float t = 0.0f;
        CK(cudaEventElapsedTime(&t, ev[0], ev[1]));
        if (rep) total += t;
    }
    cudaEventDestroy(ev[0]); cudaEventDestroy(ev[1]);
    if (r) return r;
    *ms = total / (float)reps;
    return 0;
}

int lm_read_residual(nb200_engine *h, uint32_t run, float *dst, uint32_t count) {
    LayeredEngine *e = self(h);
    if (!e->keep) return fail(NB200_EINVAL, "residuals are kept only by engines created with NB200_KEEP_RESIDUALS=1");
    if (run >= e->runs.size() || !dst || count > e->last_T * e->E) return fail(NB200_EINVAL, "bad run / count");
    CK(cudaSetDevice(e->device));
    CK(cudaMemcpyAsync(dst, e->keep + (size_t)run * e->chunk_cap * e->E, (size_t)count * 4, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    return 0;
}

// ---------------- generation on the implicit sequence ----------------
int gen_reset(LayeredEngine *e) {
    int r;
    if (e->gen_seq >= 0 && (r = lm_seq_close(reinterpret_cast<nb200_engine *>(e), (uint32_t)e->gen_seq))) return r;
    uint32_t s = 0;
    if ((r = lm_seq_open(reinterpret_cast<nb200_engine *>(e), &s))) return r;
    e->gen_seq = (int)s;
    return 0;
}

// brings the implicit sequence to `pos` tokens: pos 0 starts over; tokens between its length and pos come from ids[]
int gen_seek(LayeredEngine *e, const uint32_t *ids, uint32_t pos) {
    int r;
    if (pos == 0 || e->gen_seq < 0) { if ((r = gen_reset(e))) return r; }
    Seq &s = e->seqs[e->gen_seq];
    if (pos < s.len) return fail(NB200_EINVAL, "position %u lies before the %u tokens this engine has consumed (positions arrive in order; 0 starts over)", pos, s.len);
    if (pos > s.len) {
        if (!ids) return fail(NB200_EINVAL, "position %u skips tokens %u..%u", pos, s.len, pos - 1);
        const uint32_t n = pos - s.len;
        if ((r = check_tokens(e, ids + s.len, n))) return r;
        if (n > e->max_tokens) return fail(NB200_EINVAL, "portion longer than the engine's max_tokens");
        CK(cudaMemcpyAsync(e->ids_dev, ids + s.len, (size_t)n * 4, cudaMemcpyHostToDevice, e->stream));
        CK(cudaStreamSynchronize(e->stream));
        if ((r = step_dev(e, (uint32_t)e->gen_seq, e->ids_dev, n, nullptr, 0, nullptr))) return r;
    }
    return 0;
}

// one token of the implicit sequence; its logits end in e->logits[0..V)
int gen_token(LayeredEngine *e, uint32_t token) {
    int r;
    if (token >= e->V) return fail(NB200_EINVAL, "token/pos out of range");
    const uint32_t seq = (uint32_t)e->gen_seq;
    Seq &s = e->seqs[seq];
    if ((r = reserve_pages(e, seq, s.len + 1))) return r;
    CK(cudaMemcpyAsync(e->ids_dev + s.len, &token, 4, cudaMemcpyHostToDevice, e->stream));
    CK(cudaMemcpyAsync(e->dpos, &s.len, 4, cudaMemcpyHostToDevice, e->stream));
    if ((r = decode_step(e, seq))) return r;
    s.len += 1;
    return 0;
}

int lm_forward(nb200_engine *h, uint32_t token, uint32_t pos, uint32_t is_causal) {
    LayeredEngine *e = self(h);
    if (!is_causal) return fail(NB200_EINVAL, "this model family is causal only");
    CK(cudaSetDevice(e->device));
    int r;
    if ((r = gen_seek(e, nullptr, pos)) || (r = gen_token(e, token))) return r;
    CK(cudaStreamSynchronize(e->stream));
    return 0;
}

int lm_read_logits(nb200_engine *h, float *out) {
    LayeredEngine *e = self(h);
    if (!out) return fail(NB200_EINVAL, "null argument");
    CK(cudaSetDevice(e->device));
    CK(cudaMemcpyAsync(out, e->logits, (size_t)e->V * 4, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    return 0;
}

int mark_seen(LayeredEngine *e, const uint32_t *ids, uint32_t pos) {
    CK(cudaMemsetAsync(e->seen, 0, e->V, e->stream));
    if (!pos) return 0;
    int r;
    if ((r = check_tokens(e, ids, pos))) return r;
    if (pos > e->max_tokens) return fail(NB200_EINVAL, "more ids than the engine's max_tokens");
    CK(cudaMemcpyAsync(e->ids_dev + 8, ids, (size_t)pos * 4, cudaMemcpyHostToDevice, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    k_mark<<<ew_grid(pos), 256, 0, e->stream>>>(e->seen, e->ids_dev + 8, pos);
    CK(cudaGetLastError());
    e->launches++;
    return 0;
}

int lm_next_greedy(nb200_engine *h, const uint32_t *ids, uint32_t pos, int is_prefilling, float penalty, uint32_t *next) {
    LayeredEngine *e = self(h);
    if (!ids || !next) return fail(NB200_EINVAL, "null argument");
    CK(cudaSetDevice(e->device));
    int r;
    if ((r = gen_seek(e, ids, pos)) || (r = gen_token(e, ids[pos]))) return r;
    const float pen = is_prefilling ? 1.0f : penalty;
    if (pen != 1.0f && (r = mark_seen(e, ids, pos))) return r;
    PickArgs p{e->logits, e->seen, e->seen, e->ids_dev, e->next_dev, e->V, 0, 0, pen, 0, nullptr};
    if ((r = launch<PickArgs>(e, k_pick, dim3(1), dim3(1024), 0, p))) return r;
    CK(cudaMemcpyAsync(e->tok_host, e->next_dev, 4, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    *next = is_prefilling ? ids[pos + 1] : *e->tok_host;
    return 0;
}

int lm_next_sampled(nb200_engine *h, const uint32_t *ids, uint32_t pos, float penalty, float temperature, float top_p, float coin, uint32_t *next, uint32_t *top6) {
    LayeredEngine *e = self(h);
    if (!ids || !next) return fail(NB200_EINVAL, "null argument");
    if (!(temperature > 0.0f)) return fail(NB200_EINVAL, "temperature must be > 0 (use nb200_next_greedy for 0)");
    CK(cudaSetDevice(e->device));
    if (!e->samp_ws) {
        const size_t bytes = nb::sample_workspace_bytes(e->V, &e->samp_cub);
        DM(e->samp_ws, bytes);
        CK(cudaHostAlloc(&e->samp_host, 64, cudaHostAllocDefault));
    }
    int r;
    if ((r = gen_seek(e, ids, pos)) || (r = gen_token(e, ids[pos]))) return r;
    if (penalty != 1.0f) {      // k_pick applies the penalty to the logits in place; its greedy choice is not used
        if ((r = mark_seen(e, ids, pos))) return r;
        PickArgs p{e->logits, e->seen, e->seen, e->ids_dev, e->next_dev, e->V, 0, 0, penalty, 0, nullptr};
        if ((r = launch<PickArgs>(e, k_pick, dim3(1), dim3(1024), 0, p))) return r;
    }
    uint32_t *out_dev = nullptr;
    CK(nb::sample_top_p_launch(e->samp_ws, e->samp_cub, e->logits, e->V, temperature, top_p, coin, nullptr, &out_dev, e->stream));
    e->launches += 3;
    CK(cudaMemcpyAsync(e->samp_host, out_dev, 32, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    *next = e->samp_host[0];
    if (top6) for (int i = 0; i < 6; i++) top6[i] = e->samp_host[1 + i];
    return 0;
}

// prompt ids[0..n_prompt) -> greedy ids[n_prompt..n_total); positions 0..n_prompt-2 run as one prefill portion, the rest token by
// token with the choice fed back on the device (no host round trip per token)
int lm_decode_greedy(nb200_engine *h, uint32_t *ids, uint32_t n_prompt, uint32_t n_total, float penalty, float *prefill_ms, float *device_ms) {
    LayeredEngine *e = self(h);
    if (!ids) return fail(NB200_EINVAL, "null argument");
    if (n_prompt < 1 || n_total < n_prompt || n_total > e->max_tokens + 1) return fail(NB200_EINVAL, "bad n_prompt/n_total");
    int r;
    if ((r = check_tokens(e, ids, n_prompt))) return r;
    CK(cudaSetDevice(e->device));
    if ((r = gen_reset(e))) return r;
    const uint32_t seq = (uint32_t)e->gen_seq;
    Seq &s = e->seqs[seq];
    if ((r = reserve_pages(e, seq, n_total))) return r;
    struct Events { cudaEvent_t ev[3] = {nullptr, nullptr, nullptr}; ~Events() { for (auto v : ev) if (v) cudaEventDestroy(v); } } evs;
    for (auto &v : evs.ev) CK(cudaEventCreate(&v));
    CK(cudaMemcpyAsync(e->ids_dev, ids, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, e->stream));
    CK(cudaMemsetAsync(e->seen, 0, e->V, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    CK(cudaEventRecord(evs.ev[0], e->stream));
    if (n_prompt > 1) {
        if ((r = step_dev(e, seq, e->ids_dev, n_prompt - 1, nullptr, 0, nullptr))) return r;
        if (penalty != 1.0f) { k_mark<<<ew_grid(n_prompt - 1), 256, 0, e->stream>>>(e->seen, e->ids_dev, n_prompt - 1); CK(cudaGetLastError()); e->launches++; }
    }
    CK(cudaEventRecord(evs.ev[1], e->stream));
    const uint64_t before = e->launches;
    const uint32_t first = n_prompt - 1;
    CK(cudaMemcpyAsync(e->dpos, &first, 4, cudaMemcpyHostToDevice, e->stream));
    for (uint32_t pos = first; pos + 1 < n_total; pos++) {      // the position and the chosen token move on the device (k_pick)
        if ((r = decode_step(e, seq))) return r;
        s.len = pos + 1;
        PickArgs p{e->logits, e->seen, e->seen, e->ids_dev, e->next_dev, e->V, pos, n_prompt, penalty, 1, e->dpos};
        if ((r = launch<PickArgs>(e, k_pick, dim3(1), dim3(1024), 0, p))) return r;
    }
    if (n_total > n_prompt) e->launches_per_token = (uint32_t)((e->launches - before) / (n_total - n_prompt));
    CK(cudaEventRecord(evs.ev[2], e->stream));
    CK(cudaMemcpyAsync(ids, e->ids_dev, (size_t)n_total * 4, cudaMemcpyDeviceToHost, e->stream));
    CK(cudaStreamSynchronize(e->stream));
    float a = 0, b = 0;
    CK(cudaEventElapsedTime(&a, evs.ev[0], evs.ev[1]));
    CK(cudaEventElapsedTime(&b, evs.ev[1], evs.ev[2]));
    if (prefill_ms) *prefill_ms = a;
    if (device_ms) *device_ms = b;
    return 0;
}

int lm_get_config(const nb200_engine *h, nb200_config *c) {
    const LayeredEngine *e = self(h);
    memset(c, 0, sizeof *c);
    c->arch = NB200_ARCH_LAYERED; c->quant = e->f32 ? 0x00u : 0x16u;      // 0x16: bfloat16 weights as stored
    c->vocab_size = e->V; c->n_layer = (uint32_t)e->runs.size(); c->n_embd = e->E; c->max_seq_len = e->max_tokens; c->tp_size = 1;
    c->reserved[0] = e->use_graph ? 1u : 0u; c->reserved[3] = (uint32_t)e->layers.size(); c->reserved[4] = e->chunk_cap; c->reserved[5] = e->n_pages; c->reserved[6] = (uint32_t)e->free_pages.size();
    return 0;
}

void lm_destroy(nb200_engine *h) {
    LayeredEngine *e = self(h);
    cudaSetDevice(e->device);
    if (e->stream) cudaStreamSynchronize(e->stream);
    for (cudaGraphExec_t g : e->graphs) if (g) cudaGraphExecDestroy(g);
    for (void *p : e->allocs) cudaFree(p);
    if (e->tok_host) cudaFreeHost(e->tok_host);
    if (e->samp_host) cudaFreeHost(e->samp_host);
    if (e->ev_fork) cudaEventDestroy(e->ev_fork);
    if (e->ev_join) cudaEventDestroy(e->ev_join);
    if (e->ev_join2) cudaEventDestroy(e->ev_join2);
    if (e->side) cudaStreamDestroy(e->side);
    if (e->side2) cudaStreamDestroy(e->side2);
    if (e->stream) cudaStreamDestroy(e->stream);
    delete e;
}

const nb::EngineOps kLayeredOps = {lm_destroy, lm_get_config, lm_forward, lm_read_logits, lm_next_greedy, lm_next_sampled, lm_decode_greedy,
                                   lm_seq_open, lm_seq_close, lm_step, lm_read_residual, lm_step_timed};


int create(LayeredEngine *e, const nb::ModelDir *dir, uint32_t max_tokens) {
    const nb::Json &cfg = dir->config;
    const nb::Json *layers = cfg.get("layers");
    double eps;
    if (!u32_of(&cfg, "vocab", &e->V) || !u32_of(&cfg, "width", &e->E) || !layers || layers->t != nb::Json::Arr || layers->arr.empty() || !cfg.get("norm") || !cfg.get("norm")->number("eps", &eps))
        return fail(NB200_EINVAL, "config.json needs vocab, width, norm.eps and a non-empty list \"layers\"");
    if (!e->V || !e->E) return fail(NB200_EINVAL, "zero vocab or width");
    e->eps = (float)eps;
    const uint32_t E = e->E, NL = (uint32_t)layers->arr.size();
    Loader ld{e, dir};
    int r;
    const nb::Json *arch = cfg.get("architecture");
    const std::string design = arch && arch->t == nb::Json::Str ? arch->str : "";
    e->form = design == "Rakarax" || design == "Gokinex" ? FORM_SANDWICH : (design == "Vumunex" ? FORM_HYPER : FORM_PARALLEL_SHIFT);
    e->norm_kind = design == "Gokinex" ? NORM_DYT : NORM_RMS_ZERO;
    if ((r = ld.stacked({"embed"}, {e->V}, E, &e->embed)) || (r = ld.stacked({"head"}, {e->V}, E, &e->head))) return r;
    e->layers.resize(NL);
    if (e->norm_kind == NORM_DYT) {
        // embedding: a fixed scale on the token row and, optionally, a table of hashed (previous, current) pairs with one more row
        // for the first token of a sequence
        const nb::Json *emb = cfg.get("embedding");
        double sc = 1.0;
        if (emb && emb->t == nb::Json::Obj && emb->present("scale") && !emb->number("scale", &sc)) return fail(NB200_EINVAL, "embedding.scale must be a number");
        e->emb_scale = (float)sc;
        if (emb && emb->t == nb::Json::Obj && emb->present("bigram")) {
            const nb::Json *bg = emb->get("bigram");
            if (!u32_of(bg, "buckets", &e->buckets) || !u32_of(bg, "mul_prev", &e->mul_prev) || !u32_of(bg, "mul_cur", &e->mul_cur) || !e->buckets)
                return fail(NB200_EINVAL, "embedding.bigram needs buckets > 0, mul_prev and mul_cur");
            if ((r = ld.stacked({"bigram"}, {(uint64_t)e->buckets + 1u}, E, &e->pairs))) return r;
        }
        if ((r = load_dyt(ld, "embed.norm", E, &e->embed_norm)) || (r = load_dyt(ld, "final.norm", E, &e->final_dyt))) return r;
        // positions a sequence can reach: every page the state manager will own (the position tables cover them all)
        const uint32_t page_tokens = ((max_tokens + kPage - 1) / kPage + std::max(1u, env_u32("NB200_MAX_SEQS", 8))) * kPage;
        for (uint32_t i = 0; i < NL; i++) {
            Run q; q.layer = i; e->runs.push_back(q);
            const nb::Json &lj = layers->arr[i];
            Layer &L = e->layers[i];
            const std::string p = "l" + std::to_string(i) + ".";
            const nb::Json *type = lj.get("type"), *mixer = lj.get("mixer");
            if (!type || type->t != nb::Json::Str || !mixer || mixer->t != nb::Json::Obj) return fail(NB200_EINVAL, "layer %u needs \"type\" and \"mixer\"", i);
            if ((r = load_dyt(ld, p + "norm1", E, &L.d1)) || (r = load_dyt(ld, p + "norm1b", E, &L.d1b))) return r;
            if (type->str == "attention") { L.type = MIX_DIFF_ATTN; r = load_diff_attn(ld, mixer, p + "mix.", &L, E, page_tokens, e->layers, i); }
            else if (type->str == "mamba2") { L.type = MIX_SSD; r = load_ssd(ld, mixer, p + "mix.", &L, E); }
            else return fail(NB200_EINVAL, "layer %u: mixer type \"%s\" is not known", i, type->str.c_str());
            if (r) return r;
            if (lj.present("mlp")) {
                const nb::Json *f = lj.get("mlp"), *kind = f->get("kind");
                if ((r = load_dyt(ld, p + "norm2", E, &L.d2)) || (r = load_dyt(ld, p + "norm2b", E, &L.d2b))) return r;
                if (kind && kind->t == nb::Json::Str && kind->str == "dense") r = load_glu_dense(ld, f, p + "mlp.", &L, E);
                else if (kind && kind->t == nb::Json::Str && kind->str == "moe") r = load_moe_scored(ld, f, p + "mlp.", &L, E);
                else return fail(NB200_EINVAL, "layer %u: feed-forward kind \"%s\" is not known", i, kind && kind->t == nb::Json::Str ? kind->str.c_str() : "?");
                if (r) return r;
            }
        }
    } else if (e->form == FORM_HYPER) {
        const nb::Json *emb = cfg.get("embedding");
        double sc = 1.0, mult = 1.0;
        if (emb && emb->t == nb::Json::Obj && emb->present("scale") && !emb->number("scale", &sc)) return fail(NB200_EINVAL, "embedding.scale must be a number");
        if (cfg.present("residual_mult") && !cfg.number("residual_mult", &mult)) return fail(NB200_EINVAL, "residual_mult must be a number");
        e->emb_scale = (float)sc; e->res_mult = (float)mult;
        if (cfg.present("streams") && (!u32_of(&cfg, "streams", &e->S) || !e->S || e->S > kMaxStreams)) return fail(NB200_EINVAL, "streams must be between 1 and %u", kMaxStreams);
        if ((r = ld.vec("final.norm", {E}, &e->final_norm))) return r;
        const uint32_t page_tokens = ((max_tokens + kPage - 1) / kPage + std::max(1u, env_u32("NB200_MAX_SEQS", 8))) * kPage;      // every position the cache pages can hold
        for (uint32_t i = 0; i < NL; i++) {
            const nb::Json &lj = layers->arr[i];
            Layer &L = e->layers[i];
            const std::string p = "l" + std::to_string(i) + ".";
            const nb::Json *type = lj.get("type"), *mixer = lj.get("mixer");
            if (!type || type->t != nb::Json::Str || !mixer || mixer->t != nb::Json::Obj) return fail(NB200_EINVAL, "layer %u needs \"type\" and \"mixer\"", i);
            if ((r = ld.vec(p + "norm1", {E}, &L.ln1)) || (r = load_hc(ld, p + "hc1.", e->S, &L.hc1))) return r;
            if (dir->tensors.count(p + "ls1") && (r = ld.vec(p + "ls1", {E}, &L.ls1))) return r;
            // both kinds are one mechanism: what a kind has (rotated part, window, sink, gate) shows in its config entry and tensors
            if (type->str == "latent_attention" || type->str == "latent_attention_2") { L.type = MIX_LATENT_ATTN; r = load_latent_attn_direct(ld, mixer, p + "mix.", &L, E, page_tokens); }
            else return fail(NB200_EINVAL, "layer %u: mixer type \"%s\" is not known", i, type->str.c_str());
            if (r) return r;
            if (lj.present("mlp")) {
                const nb::Json *f = lj.get("mlp"), *kind = f->get("kind");
                if ((r = ld.vec(p + "norm2", {E}, &L.ln2)) || (r = load_hc(ld, p + "hc2.", e->S, &L.hc2))) return r;
                if (dir->tensors.count(p + "ls2") && (r = ld.vec(p + "ls2", {E}, &L.ls2))) return r;
                if (kind && kind->t == nb::Json::Str && kind->str == "dense") r = load_dense_gelu(ld, f, p + "mlp.", &L, E);
                else if (kind && kind->t == nb::Json::Str && kind->str == "moe") r = load_moe_scored(ld, f, p + "mlp.", &L, E, true);
                else return fail(NB200_EINVAL, "layer %u: feed-forward kind \"%s\" is not known", i, kind && kind->t == nb::Json::Str ? kind->str.c_str() : "?");
                if (r) return r;
            }
        }
    } else if (e->form == FORM_SANDWICH) {
        auto pt = dir->tensors.find("pos");
        if (pt == dir->tensors.end() || pt->second.shape.size() != 2 || pt->second.shape[0] == 0) return fail(NB200_EINVAL, "model.safetensors has no position table \"pos\" [positions, width]");
        e->max_pos = (uint32_t)pt->second.shape[0];
        if ((r = ld.stacked({"pos"}, {e->max_pos}, E, &e->pos_table)) || (r = ld.vec("final.norm", {E}, &e->final_norm))) return r;
        // a layer with "weights_of": j runs layer j's tensors with cache and state of its own
        std::vector<uint32_t> owner(NL);
        for (uint32_t i = 0; i < NL; i++) {
            owner[i] = i;
            for (uint32_t hops = 0; layers->arr[owner[i]].present("weights_of"); hops++) {          // a named layer may itself name another
                uint32_t j = 0;
                if (!u32_of(&layers->arr[owner[i]], "weights_of", &j) || j >= NL || hops > NL) return fail(NB200_EINVAL, "layer %u: weights_of must lead to a layer with weights of its own", i);
                owner[i] = j;
            }
        }
        for (uint32_t i = 0; i < NL; i++) {
            Run q; q.layer = owner[i]; e->runs.push_back(q);
            if (owner[i] != i) continue;
            const nb::Json &lj = layers->arr[i];
            Layer &L = e->layers[i];
            const std::string p = "l" + std::to_string(i) + ".";
            const nb::Json *type = lj.get("type"), *mixer = lj.get("mixer");
            if (!type || type->t != nb::Json::Str || !mixer || mixer->t != nb::Json::Obj) return fail(NB200_EINVAL, "layer %u needs \"type\" and \"mixer\"", i);
            if ((r = ld.vec(p + "norm1", {E}, &L.n1)) || (r = ld.vec(p + "norm1b", {E}, &L.n1b))) return r;
            if (type->str == "retention") { L.type = MIX_RETENTION; r = load_retention(ld, mixer, p + "mix.", &L, E, e->max_pos); }
            else if (type->str == "parallel") { L.type = MIX_WINDOW_SSM; r = load_window_ssm(ld, mixer, p + "mix.", &L, E); }
            else return fail(NB200_EINVAL, "layer %u: mixer type \"%s\" is not known", i, type->str.c_str());
            if (r) return r;
            if (lj.present("mlp")) {
                const nb::Json *f = lj.get("mlp"), *kind = f->get("kind");
                if (!kind || kind->t != nb::Json::Str || kind->str != "dense") return fail(NB200_EINVAL, "layer %u: feed-forward kind \"%s\" is not known here", i, kind && kind->t == nb::Json::Str ? kind->str.c_str() : "?");
                if ((r = ld.vec(p + "norm2", {E}, &L.n2)) || (r = ld.vec(p + "norm2b", {E}, &L.n2b)) || (r = load_dense(ld, f, p + "mlp.", &L, E))) return r;
            }
        }
    } else {
        if ((r = ld.vec("final.norm", {}, &e->final_norm))) return r;
        for (uint32_t i = 0; i < NL; i++) {
            const nb::Json &lj = layers->arr[i];
            Layer &L = e->layers[i];
            const std::string p = "l" + std::to_string(i) + ".";
            const nb::Json *type = lj.get("type"), *mixer = lj.get("mixer");
            if (!type || type->t != nb::Json::Str || !mixer || mixer->t != nb::Json::Obj) return fail(NB200_EINVAL, "layer %u needs \"type\" and \"mixer\"", i);
            if ((r = ld.vec(p + "norm1", {}, &L.norm1)) || (r = ld.vec(p + "shift", {E}, &L.shift))) return r;
            if (type->str == "rglru") { L.type = MIX_RGLRU; r = load_rglru(ld, mixer, p + "mix.", &L, E); }
            else if (type->str == "latent_attention") { L.type = MIX_LATENT_ATTN; r = load_latent_attn(ld, mixer, p + "mix.", &L, E); }
            else return fail(NB200_EINVAL, "layer %u: mixer type \"%s\" is not known", i, type->str.c_str());
            if (r) return r;
            if (lj.present("mlp")) {
                if ((r = ld.vec(p + "norm2", {}, &L.norm2)) || (r = load_moe(ld, lj.get("mlp"), p + "mlp.", &L, E))) return r;
            }
        }
    }
    if (e->form == FORM_PARALLEL_SHIFT || e->form == FORM_HYPER) {
        // order of the layer runs: a span may run several times in a row (the parallel form adds the embedding output again before every pass but the first)
        uint32_t lo = 0, hi = 0, times = 1;
        if (cfg.present("loop")) {
            const nb::Json *lp = cfg.get("loop");
            if (!u32_of(lp, "start", &lo) || !u32_of(lp, "stop", &hi) || !u32_of(lp, "times", &times) || lo > hi || hi > NL || times < 1) return fail(NB200_EINVAL, "loop needs 0 <= start <= stop <= layers and times >= 1");
        }
        for (uint32_t i = 0; i < lo; i++) { Run q; q.layer = i; e->runs.push_back(q); }
        for (uint32_t p = 0; p < times; p++) for (uint32_t i = lo; i < hi; i++) { Run q; q.layer = i; q.add_embed = e->form == FORM_PARALLEL_SHIFT && p > 0 && i == lo; e->runs.push_back(q); if (q.add_embed) e->keep_x0 = true; }
        for (uint32_t i = hi; i < NL; i++) { Run q; q.layer = i; e->runs.push_back(q); }
    }

    // state manager: slots and pages
    e->max_tokens = max_tokens;
    e->max_seqs = std::max(1u, env_u32("NB200_MAX_SEQS", 8));
    e->chunk_cap = std::max(1u, std::min(max_tokens, env_u32("NB200_CHUNK", 1024)));
    e->n_pages = (max_tokens + kPage - 1) / kPage + e->max_seqs;
    size_t off = 0;
    if (e->buckets) { e->st_tok = off; off += 4; }      // the sequence's last token + 1, one word (the pair table's hash needs it)
    for (Run &q : e->runs) {
        const Layer &L = e->layers[q.layer];
        if (e->form == FORM_PARALLEL_SHIFT) { q.st_prev = off; off += E; }
        switch (L.type) {
            case MIX_DIFF_ATTN:      // rows of [rotated keys of both maps | values]; a layer that reads another layer's rows has none
                if (L.kv_from >= 0) { q.cache = e->runs[L.kv_from].cache; break; }
                DM(q.cache, (size_t)e->n_pages * kPage * L.RL * 4);
                CK(cudaMemset(q.cache, 0, (size_t)e->n_pages * kPage * L.RL * 4));
                break;
            case MIX_SSD:            // the convolution's tail over [x | B | C] and the state [head][value column][state coordinate]
                q.st_conv = off; off += (size_t)(L.m_taps - 1) * (L.H * L.vdim + 2 * L.G * L.mN);
                q.st_S = off; off += (size_t)L.H * L.vdim * L.mN;
                break;
            case MIX_RGLRU: q.st_S = off; off += L.C; q.st_conv = off; off += (size_t)(L.taps - 1) * L.C; break;
            case MIX_LATENT_ATTN:      // rows of [latent | rotated key part | padding]
                DM(q.cache, (size_t)e->n_pages * kPage * L.RS * 4);
                CK(cudaMemset(q.cache, 0, (size_t)e->n_pages * kPage * L.RS * 4));
                break;
            case MIX_RETENTION: q.st_S = off; off += (size_t)L.H * L.vdim * L.dim; break;
            default:          // window attention + selective scan: the tails of both convolutions, the scan state, a cache of key/value rows
                q.st_conv = off; off += (size_t)(L.a_taps - 1) * (L.H + L.G) * L.dim;
                q.st_conv2 = off; off += (size_t)(L.m_taps - 1) * L.mC;
                q.st_S = off; off += (size_t)L.mC * L.mN;
                DM(q.cache, (size_t)e->n_pages * kPage * L.RL * 4);
                CK(cudaMemset(q.cache, 0, (size_t)e->n_pages * kPage * L.RL * 4));
        }
    }
    e->slot_floats = (off + 3) & ~(size_t)3;
    DM(e->state, (size_t)e->max_seqs * e->slot_floats * 4);
    DM(e->state_bak, e->slot_floats * 4);
    DM(e->table, (size_t)e->max_seqs * e->n_pages * 4);
    CK(cudaMemset(e->table, 0, (size_t)e->max_seqs * e->n_pages * 4));
    e->seqs.resize(e->max_seqs);
    for (uint32_t p = e->n_pages; p > 0; p--) e->free_pages.push_back(p - 1);

    // scratch for one chunk
    const size_t T = e->chunk_cap;
    uint32_t mC = 0, mZ = 0, mQR = 0, mQ = 0, mHR = 0, mOV = 0, mNE = 0, mTop = 0, mFF = 0, mSFF = 0;
    uint32_t sP = 0, sQK = 0, sXC = 0, sA = 0, sRO = 0, sDBC = 0, sF = 0;
    uint32_t sDP = 0, sDT = 0, sXC2 = 0, sY = 0, sF2 = 0; size_t sSS = 0, diff_smem[4] = {0, 0, 0, 0};      // differential attention, state-space duality, gated feed-forward
    size_t win_smem[4] = {0, 0, 0, 0};      // most shared memory any layer asks of the window-attention instances, per value-column count
    for (const Run &q : e->runs) {
        const Layer &L = e->layers[q.layer];
        if (L.type == MIX_RETENTION) { sP = std::max(sP, 2 * L.H * (L.dim + L.vdim)); sA = std::max(sA, L.H * L.vdim); sRO = std::max(sRO, L.H * L.vdim); }
        if (L.type == MIX_WINDOW_SSM) {
            sP = std::max(sP, (2 * L.H + L.G) * L.dim + 2 * L.mC); sQK = std::max(sQK, (L.H + L.G) * L.dim); sXC = std::max(sXC, L.mC); sA = std::max(sA, L.H * L.dim);
            sDBC = std::max(sDBC, L.mR + 2 * L.mN);
            const uint32_t qt = win_attn_qt(L);
            if (!qt) return fail(NB200_EINVAL, "window attention with %u heads of %u does not fit the attention kernel's shared memory", L.H, L.dim);
            size_t &sm = win_smem[L.dim <= 32 ? 0 : L.dim <= 64 ? 1 : L.dim <= 128 ? 2 : 3];
            sm = std::max(sm, std::max(win_attn_smem(L.H, L.dim, L.RL, qt), win_attn_smem(L.H, L.dim, L.RL, 1)));
        }
        if (L.ff_kind == FF_DENSE_POLY || L.ff_kind == FF_DENSE_GELU) sF = std::max(sF, L.ff);
        if (L.type == MIX_DIFF_ATTN) {
            sP = std::max(sP, L.H * 2 * L.dim + (L.kv_from < 0 ? L.G * (2 * L.dim + L.vdim) : 0u)); sA = std::max(sA, L.H * L.vdim);
            sDP = std::max(sDP, L.H * 2 * (L.vdim + 2)); sDT = std::max(sDT, (L.H + L.a_hpb1 - 1) / L.a_hpb1);
            const bool vec = diff_attn_vec(L.dim, L.vdim, L.H * 2 * L.dim + (L.kv_from < 0 ? L.G * (2 * L.dim + L.vdim) : 0u));
            size_t &sm = diff_smem[diff_vch(L.vdim)];
            sm = std::max(sm, std::max(diff_attn_smem(L.dim, L.vdim, L.a_ngk, L.a_qt, L.a_hpb, vec), diff_attn_smem(L.dim, L.vdim, L.a_ngk1, 1, L.a_hpb1, vec)));
        }
        if (L.type == MIX_SSD) {
            const uint32_t inner = L.H * L.vdim, XW = inner + 2 * L.G * L.mN;
            sP = std::max(sP, inner + XW + L.H); sXC2 = std::max(sXC2, XW); sY = std::max(sY, inner); sA = std::max(sA, inner);
            sSS = std::max(sSS, (size_t)inner * L.mN);
        }
        if (L.ff_kind == FF_DENSE_GLU) { sF = std::max(sF, 2 * L.ff); sF2 = std::max(sF2, L.ff); }
    }
    if (diff_smem[0] > 48 * 1024 && (r = diff_attn_optin_v<1>((int)diff_smem[0]))) return r;
    if (diff_smem[1] > 48 * 1024 && (r = diff_attn_optin_v<2>((int)diff_smem[1]))) return r;
    if (diff_smem[2] > 48 * 1024 && (r = diff_attn_optin_v<4>((int)diff_smem[2]))) return r;
    if (diff_smem[3] > 48 * 1024 && (r = diff_attn_optin_v<8>((int)diff_smem[3]))) return r;
    if (sDP) {
        DM(e->b_dpart, (size_t)kGemvMaxM * kSplitMax * sDP * 4);
        DM(e->b_dtick, (size_t)kGemvMaxM * sDT * 4);
        CK(cudaMemset(e->b_dtick, 0, (size_t)kGemvMaxM * sDT * 4));
    }
    if (sSS) DM(e->b_sseg, (size_t)kRetSegs * sSS * 4);
    if (sXC2) DM(e->b_sdx, T * sXC2 * 4);
    if (sY) DM(e->b_sdy, T * sY * 4);
    if (sF2) DM(e->b_f2, T * sF2 * 4);
    if (sQK && ((r = sel_scan_optin<1>()) || (r = sel_scan_optin<2>()) || (r = sel_scan_optin<4>()) || (r = sel_scan_optin<8>()) || (r = sel_scan_optin<16>()) || (r = sel_scan_optin<32>()))) return r;
    if (win_smem[0] > 48 * 1024 && (r = win_attn_optin_v<1>((int)win_smem[0]))) return r;
    if (win_smem[1] > 48 * 1024 && (r = win_attn_optin_v<2>((int)win_smem[1]))) return r;
    if (win_smem[2] > 48 * 1024 && (r = win_attn_optin_v<4>((int)win_smem[2]))) return r;
    if (win_smem[3] > 48 * 1024 && (r = win_attn_optin_v<8>((int)win_smem[3]))) return r;
    if (sP) DM(e->b_p, T * sP * 4);
    if (sQK) DM(e->d2, T * E * 4);
    if (sRO) {
        uint32_t mH = 0; size_t mS = 0;
        for (const Run &q : e->runs) { const Layer &L = e->layers[q.layer]; if (L.type == MIX_RETENTION) { mH = std::max(mH, L.H); mS = std::max(mS, (size_t)L.H * L.vdim * L.dim); } }
        DM(e->b_rseg, (size_t)kRetSegs * mS * 4);
        DM(e->b_rtick, (size_t)mH * 4);
        CK(cudaMemset(e->b_rtick, 0, (size_t)mH * 4));
    }
    if (sQK) {
        uint32_t mPart = 0;
        for (const Run &q : e->runs) { const Layer &L = e->layers[q.layer]; if (L.type == MIX_WINDOW_SSM) mPart = std::max(mPart, L.H * (L.dim + 2)); }
        DM(e->b_wpart, (size_t)kGemvMaxM * kSplitMax * mPart * 4);
        DM(e->b_wtick, (size_t)kGemvMaxM * 4);
        CK(cudaMemset(e->b_wtick, 0, (size_t)kGemvMaxM * 4));
    }
    if (sQK) { DM(e->b_qk, T * sQK * 4); DM(e->b_xc, T * sXC * 4); DM(e->b_dbc, T * sDBC * 4); DM(e->b_dt, T * sXC * 4); DM(e->b_y, T * sXC * 4); }
    if (sA) DM(e->b_a, T * sA * 4);
    if (sRO) DM(e->b_ro, T * sRO * 4);
    if (sF) DM(e->b_f, T * sF * 4);
    uint32_t mFF2 = 0, mSFF2 = 0;      // scored experts: [gate | up] rows of a prefill portion
    for (const Layer &L : e->layers) {
        if (L.type == MIX_RGLRU) mC = std::max(mC, L.C);
        else if (L.type == MIX_LATENT_ATTN) {
            mZ = std::max(mZ, L.QR ? L.QR + L.R : L.H * (L.dim + L.RD + L.vdim) + L.R + L.RD); mQR = std::max(mQR, L.QR); mQ = std::max(mQ, L.H * L.dim);
            mHR = std::max(mHR, L.H * L.RS); mOV = std::max(mOV, L.H * L.vdim);
        }
        if (L.ff_kind == FF_MOE || L.ff_kind == FF_MOE_SCORED) { mNE = std::max(mNE, L.NE + 1u); mTop = std::max(mTop, L.top); mFF = std::max(mFF, L.top * L.ff); mSFF = std::max(mSFF, L.sff); }
        if (L.ff_kind == FF_MOE_SCORED) { mFF2 = std::max(mFF2, 2 * L.top * L.ff); mSFF2 = std::max(mSFF2, 2 * L.sff); }
    }
    if (e->form == FORM_HYPER) DM(e->xs, (size_t)e->S * T * E * 4);
    DM(e->x, T * E * 4); DM(e->hm, T * E * 4); DM(e->h2, T * E * 4); DM(e->d, T * E * 4);
    if (e->keep_x0) DM(e->x0, T * E * 4);
    if (mC) { DM(e->b_yx, T * 2 * mC * 4); DM(e->b_u, T * mC * 4); DM(e->b_g, T * 2 * mC * 4); DM(e->b_sy, T * mC * 4); }
    if (mZ) {
        DM(e->b_z, T * mZ * 4); DM(e->b_cq, T * mQR * 4); DM(e->b_q, T * mQ * 4); DM(e->b_qa, T * mHR * 4); DM(e->b_ol, T * mHR * 4); DM(e->b_ov, T * mOV * 4);
        uint32_t mPart = 0, mR = 0;
        for (const Layer &L : e->layers) if (L.type == MIX_LATENT_ATTN) { mPart = std::max(mPart, L.H * (L.R + 2)); mR = std::max(mR, L.RS); }
        DM(e->b_part, (size_t)kGemvMaxM * kSplitMax * mPart * 4);
        uint32_t mHG = 0;
        for (const Layer &L : e->layers) if (L.type == MIX_LATENT_ATTN) mHG = std::max(mHG, (L.H + kAttnWarps - 1) / kAttnWarps);
        DM(e->b_tick, (size_t)kGemvMaxM * mHG * 4);
        CK(cudaMemset(e->b_tick, 0, (size_t)kGemvMaxM * mHG * 4));
        // the prefill instances by the rows they serve: kAttnQT queries per block for latents up to 256, 4 above (attn_launch)
        uint32_t mR8 = 0, mR4 = 0;
        for (const Layer &L : e->layers) if (L.type == MIX_LATENT_ATTN) { if (L.R <= 256) mR8 = std::max(mR8, L.RS); else mR4 = std::max(mR4, L.RS); }
        constexpr size_t kAttnSmemMax = 227 * 1024;
        if (std::max(attn_smem(mR8, kAttnQT), attn_smem(mR4, 4)) > kAttnSmemMax)
            return fail(NB200_EINVAL, "a cache row of %u floats (latent + rotated key part) does not fit the attention kernel's shared memory", std::max(mR8, mR4));
        if (mR8 && attn_smem(mR8, kAttnQT) > 48 * 1024 && (r = attn_optin<kAttnQT>((int)attn_smem(mR8, kAttnQT)))) return r;
        if (mR4 && attn_smem(mR4, 4) > 48 * 1024 && (r = attn_optin<4>((int)attn_smem(mR4, 4)))) return r;
        if (attn_smem(mR, 1) > 48 * 1024 && (r = attn_optin<1>((int)attn_smem(mR, 1)))) return r;
    }
    if (mNE) {
        DM(e->b_idx, T * mTop * 4); DM(e->b_wt, T * mTop * 4); DM(e->b_slot, T * mTop * 4); DM(e->b_rows, T * mTop * 4);
        DM(e->b_cnt, (size_t)mNE * 4); DM(e->b_off, ((size_t)mNE + 1) * 4); DM(e->b_fill, (size_t)mNE * 4);
        CK(cudaMemset(e->b_cnt, 0, (size_t)mNE * 4));
        DM(e->b_hb, T * mFF * 4); DM(e->b_eo, T * mTop * E * 4);
        if (mSFF) { DM(e->b_sh, T * std::max(mSFF, mSFF2) * 4); DM(e->b_so, T * E * 4); }
        if (mFF2) { DM(e->b_hg, T * mFF2 * 4); DM(e->b_wrow, T * mTop * 4); DM(e->b_sg, T * 4); }
        if (mSFF2) DM(e->b_sh2, T * mSFF * 4);
    }
    DM(e->dpos, 64); DM(e->zero_dev, 64);
    CK(cudaMemset(e->dpos, 0, 64)); CK(cudaMemset(e->zero_dev, 0, 64));
    e->graphs.assign(e->max_seqs, nullptr);
    DM(e->b_xn, (size_t)kWantBatch * E * 4); DM(e->logits, (size_t)kWantBatch * e->V * 4);
    const size_t n_ids = (size_t)e->n_pages * kPage + 16;          // a single-token step stores its token at the sequence's position: every position the pages can hold
    DM(e->ids_dev, n_ids * 4); DM(e->want_dev, kWantBatch * 4); DM(e->next_dev, 64); DM(e->seen, e->V);
    CK(cudaMemset(e->ids_dev, 0, n_ids * 4));
    CK(cudaMemset(e->seen, 0, e->V));
    if (env_u32("NB200_KEEP_RESIDUALS", 0)) DM(e->keep, e->runs.size() * T * E * 4);
    CK(cudaHostAlloc(&e->tok_host, 64, cudaHostAllocDefault));
    CK(cudaDeviceSynchronize());
    return 0;
}

}  // namespace

extern "C" int nb_family_layered_create(nb200_engine **out, const nb::ModelDir *dir, uint32_t max_tokens, int device, uint32_t flags) {
    CK(cudaSetDevice(device));
    LayeredEngine *e = new LayeredEngine();
    e->ops = &kLayeredOps;
    e->device = device; e->f32 = (flags & NB200_FLAG_F32) != 0;
    e->use_pdl = !(flags & NB200_FLAG_NO_PDL) && !env_u32("NB200_NO_PDL", 0);
    e->use_graph = !(flags & NB200_FLAG_NO_GRAPH) && !env_u32("NB200_NO_GRAPH", 0);
    e->branch_streams = !env_u32("NB200_NO_BRANCH_STREAMS", 0);
    cudaDeviceProp prop;
    cudaError_t ce = cudaGetDeviceProperties(&prop, device);
    if (ce == cudaSuccess) { e->num_sms = prop.multiProcessorCount; ce = cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking); }
    if (ce == cudaSuccess) ce = cudaStreamCreateWithFlags(&e->side, cudaStreamNonBlocking);
    if (ce == cudaSuccess) ce = cudaStreamCreateWithFlags(&e->side2, cudaStreamNonBlocking);
    if (ce == cudaSuccess) ce = cudaEventCreateWithFlags(&e->ev_join2, cudaEventDisableTiming);
    if (ce == cudaSuccess) ce = cudaEventCreateWithFlags(&e->ev_fork, cudaEventDisableTiming);
    if (ce == cudaSuccess) ce = cudaEventCreateWithFlags(&e->ev_join, cudaEventDisableTiming);
    e->cur = e->stream;
    int r = ce == cudaSuccess ? create(e, dir, max_tokens) : fail(NB200_ECUDA, "device setup failed: %s", cudaGetErrorString(ce));
    if (r) { lm_destroy(reinterpret_cast<nb200_engine *>(e)); return r; }
    *out = reinterpret_cast<nb200_engine *>(e);
    return 0;
}

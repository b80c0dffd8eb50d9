// layered_mixers2.cuh -- a third set of mechanisms of the layered runtime (layered.cu), beside layered_kernels.cuh and
// layered_mixers.cuh and under their rules: a kernel (or an epilogue) per mechanism, constants as arguments, fp32 for everything
// that is not a matrix-product operand, programmatic dependent launch at the top of every kernel, positions optionally read from a
// device word (captured decode step).
//
//   embedding            k_embed_pair (token row x scale + a hashed row for the (previous, current) token pair; the previous token
//                        lives in the sequence's state slot)
//   norms                Dyt (Dynamic Tanh: tanh(alpha u) w + b, purely elementwise), k_dyt_residual (x += dyt(sublayer output),
//                        where the output may be a mixer's, a dense feed-forward's or the sum of routed experts and a gated shared
//                        expert; the next sublayer's input norm of the updated x in the same pass), k_final_dyt
//   rotary positions     k_rope_kv (interleaved pairs (2i, 2i+1) over the first `dims` coordinates of every map of every head, angles
//                        from a table built in double precision; q in place, k and v into the sequence's cache pages)
//   attention            k_diff_attn (grouped-query differential attention: two causal softmax maps per head over the same values,
//                        o = a1 - lambda a2, unit RMS over the head, fixed output scale; key splits for short portions)
//   state-space duality  k_ssd_scan (Mamba-2: one decay per head and token, S <- a_t S + dt_t B_t x_t^T, y = S^T C_t + D x_t; fp32
//                        state [head][value column][state coordinate]; long portions as time segments side by side with
//                        k_ssd_chain between the two passes; the output leaves gated, y silu(z)), k_group_norm (unit RMS in equal parts, vector gain)
//   feed-forward         k_glu (act(s g) (s u) over [gate | up] rows, s an optional per-row scale: a routed expert whose INPUT is
//                        weighted by the router's score)
#pragma once
#include "layered_mixers.cuh"

namespace nb {
namespace lm {

// Dynamic Tanh norm: elementwise, tanh(alpha u) w[i] + b[i]
struct Dyt { const float *w, *b; float alpha; };
__device__ __forceinline__ float dyt_of(const Dyt &n, float u, uint32_t i) { return fmaf(tanhf(n.alpha * u), n.w[i], n.b[i]); }

// x[t] = dyt_norm( embed[tok_t] scale + pairs[row_t] ),  row_t = (tok_(t-1) mul_prev + tok_t mul_cur) mod buckets, or row `buckets`
// for the first token of a sequence.  *prev holds the sequence's last token + 1 (0: none yet) and moves on.  out = dyt_next(x):
// the first sublayer's input.  Tokens are read at tokens[t + *pos_ptr] in a captured decode step.  buckets 0: no pair table.
struct EmbedPairArgs {
    const uint32_t *tokens; const uint32_t *pos_ptr; const void *embed; const void *pairs; float *x; float *out; uint32_t *prev;
    uint32_t T, E, buckets, mul_prev, mul_cur; float scale; Dyt norm, next;
};
template <typename WT>
__global__ void __launch_bounds__(512) k_embed_pair(const EmbedPairArgs a) {
    pdl_enter();
    const uint32_t t = blockIdx.x, off = a.pos_ptr ? *a.pos_ptr : 0u;
    const uint32_t tok = a.tokens[t + off];
    const uint32_t before = !a.buckets ? 0u : t ? a.tokens[t - 1u + off] + 1u : *a.prev;
    if (t == 0 && a.buckets) {          // the one reader of the word is also its writer, in that order
        __syncthreads();
        if (threadIdx.x == 0) *a.prev = a.tokens[a.T - 1u + off] + 1u;
    }
    const WT *src = static_cast<const WT *>(a.embed) + (size_t)tok * a.E, *pr = nullptr;
    if (a.buckets) {
        const uint64_t row = before ? ((uint64_t)(before - 1u) * a.mul_prev + (uint64_t)tok * a.mul_cur) % a.buckets : a.buckets;
        pr = static_cast<const WT *>(a.pairs) + (size_t)row * a.E;
    }
    for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) {
        float v = wval(src + i) * a.scale;
        if (pr) v += wval(pr + i);
        v = dyt_of(a.norm, v, i);
        a.x[(size_t)t * a.E + i] = v;
        if (a.out) a.out[(size_t)t * a.E + i] = dyt_of(a.next, v, i);
    }
}

// x[t] += dyt_post(u[t]),  u = d (+ sum_j eo[slot[t][j]] in the order of the choices) (+ shared[t] sigmoid(sgate[t]));  keep
// (optional) receives the updated x;  out (optional) = dyt_pre(x), the input of the sublayer that follows.
struct DytResArgs {
    float *x; const float *d; const float *eo; const uint32_t *slot; uint32_t top; const float *shared; const float *sgate;
    Dyt post, pre; float *out; float *keep; uint32_t T, E;
};
__global__ void __launch_bounds__(256) k_dyt_residual(const DytResArgs a) {
    pdl_enter();
    const size_t total = (size_t)a.T * a.E;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / a.E), c = (uint32_t)(i % a.E);
        float u = a.d ? a.d[i] : 0.0f;
        if (a.eo) for (uint32_t j = 0; j < a.top; j++) u += a.eo[(size_t)a.slot[(size_t)t * a.top + j] * a.E + c];
        if (a.shared) u = fmaf(a.shared[i], sigmoidf_(a.sgate[t]), u);
        const float v = a.x[i] + dyt_of(a.post, u, c);
        a.x[i] = v;
        if (a.keep) a.keep[i] = v;
        if (a.out) a.out[i] = dyt_of(a.pre, v, c);
    }
}

// out[r] = dyt(x[want[r]]): the rows whose logits are asked for
__global__ void __launch_bounds__(256) k_final_dyt(const float *__restrict__ x, const uint32_t *__restrict__ want, const Dyt n, float *__restrict__ out, uint32_t E) {
    pdl_enter();
    const float *xt = x + (size_t)want[blockIdx.x] * E;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) out[(size_t)blockIdx.x * E + i] = dyt_of(n, xt[i], i);
}

// out[r][c] = act(s g) (s u),  g = gu[r][c], u = gu[r][F + c], s = row_scale[r] (1 when null); act 0: gelu (tanh form), 1: silu,
// 2: the clamped unit  min(g, limit) sigmoid(1.702 min(g, limit)) (clamp(u, -limit, limit) + 1)
struct GluArgs { const float *gu; uint32_t ld; float *out; uint32_t ldo; const float *row_scale; uint32_t rows, F, act; float limit; };
__device__ __forceinline__ float glu_of(float g, float u, float s, uint32_t act, float limit) {
    g *= s; u *= s;
    if (act == 2u) return clamped_glu(g, u, limit);
    return (act ? siluf_(g) : gelu_tanh(g)) * u;
}
__global__ void __launch_bounds__(256) k_glu(const GluArgs a) {
    pdl_enter();
    const size_t total = (size_t)a.rows * a.F;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / a.F), c = (uint32_t)(i % a.F);
        const float *row = a.gu + (size_t)r * a.ld;
        a.out[(size_t)r * a.ldo + c] = glu_of(row[c], row[a.F + c], a.row_scale ? a.row_scale[r] : 1.0f, a.act, a.limit);
    }
}

// Rotary positions and the cache write of a grouped-query attention whose heads carry `maps` score maps each.  One block per token.
// p rows: q [H][maps][D] at column 0, k [G][maps][D] at k0, v [G][VD] at v0.  The pair (2i, 2i+1), i < dims/2, of every map turns by
// the angle of tab[position][i] = (cos, sin): (u, v) -> (u cos - v sin, v cos + u sin); the other coordinates pass.  q turns in
// place; the turned k and v go to the token's cache row [G maps D keys | G VD values | padding].  has_kv 0: the layer reads another
// layer's cache and only its q turns.
struct RopeKvArgs {
    float *p; uint32_t ld, k0, v0, has_kv; float *cache; const uint32_t *table;
    uint32_t T, H, G, maps, D, VD, RL, dims, pos0; const float2 *tab; const uint32_t *pos_ptr;
};
__global__ void __launch_bounds__(256) k_rope_kv(const RopeKvArgs a) {
    pdl_enter();
    const uint32_t t = blockIdx.x, pos = a.pos0 + t + (a.pos_ptr ? *a.pos_ptr : 0u);
    const uint32_t half = a.tab ? a.dims / 2u : 0u, QM = a.H * a.maps, KM = a.G * a.maps;
    float *row = a.p + (size_t)t * a.ld;
    const float2 *cs = a.tab + (size_t)pos * half;
    for (uint32_t i = threadIdx.x; i < QM * half; i += blockDim.x) {
        float *q = row + (i / half) * a.D + 2u * (i % half);
        const float2 c = cs[i % half];
        const float u = q[0], v = q[1];
        q[0] = u * c.x - v * c.y; q[1] = v * c.x + u * c.y;
    }
    if (!a.has_kv) return;
    float *dst = a.cache + ((size_t)a.table[pos / kPage] * kPage + pos % kPage) * a.RL;
    const float *k = row + a.k0, *v = row + a.v0;
    for (uint32_t i = threadIdx.x; i < KM * half; i += blockDim.x) {
        const uint32_t o = (i / half) * a.D + 2u * (i % half);
        const float2 c = cs[i % half];
        const float u = k[o], w = k[o + 1u];
        dst[o] = u * c.x - w * c.y; dst[o + 1u] = w * c.x + u * c.y;
    }
    const uint32_t rest = a.D - 2u * half;
    for (uint32_t i = threadIdx.x; i < KM * rest; i += blockDim.x) { const uint32_t o = (i / rest) * a.D + 2u * half + i % rest; dst[o] = k[o]; }
    const uint32_t KW = KM * a.D, VW = a.G * a.VD;
    for (uint32_t i = threadIdx.x; i < a.RL - KW; i += blockDim.x) dst[KW + i] = i < VW ? v[i] : 0.0f;
}

// Grouped-query differential attention over the paged cache rows k_rope_kv writes (maps = 2).  Query head h uses key/value head
// g = h / (H / G); for query position i and key position j <= i:
//     s_m = scale q_(h,m) . k_(j,g,m),  p_m = softmax_j s_m,  a_m = sum_j p_m v_(j,g)      for the two maps m = 1, 2
//     o = a_1 - lambda a_2,   out = o / sqrt(mean(o^2) + eps) x out_scale      (mean over the head's VD values)
// grid = (query tiles of QT tokens, key splits, head groups); blockDim = 32 x heads per block, one warp per head doing both maps (they
// share every value load).  A key tile is one cache page: the slices of the kv heads this block's heads use are staged in shared
// memory; lanes = keys for the scores, = value columns for the weighted sums; online softmax in fp32.  With one split the finished
// rows are written; otherwise partial (o, m, l) triples per map, merged and finished by the block that draws the last ticket of its
// (query tile, head group).
struct DiffAttnArgs {
    const float *q; uint32_t ldq; const float *cache; const uint32_t *table; float *out;
    uint32_t T, H, G, D, VD, RL, pos0; float scale, lambda, out_scale, eps; const uint32_t *pos_ptr;
    uint32_t nsplit; float *part; uint32_t *tickets; uint32_t ngk;      // ngk: the most kv heads any block stages
};
__host__ __device__ inline bool diff_attn_vec(uint32_t D, uint32_t VD, uint32_t ldq) { return ((D | VD | ldq) & 3u) == 0; }
__host__ __device__ inline uint32_t diff_attn_ldk(uint32_t kw, bool vec) { return vec ? (((kw >> 2) & 1u) ? kw : kw + 4u) : (kw | 1u); }
// kv heads staged by a block of hpb consecutive query heads
inline uint32_t diff_attn_ngk(uint32_t H, uint32_t G, uint32_t hpb) {
    const uint32_t rep = H / G; uint32_t m = 1;
    for (uint32_t h0 = 0; h0 < H; h0 += hpb) m = std::max(m, (std::min(H, h0 + hpb) - 1u) / rep - h0 / rep + 1u);
    return m;
}
inline size_t diff_attn_smem(uint32_t D, uint32_t VD, uint32_t ngk, uint32_t qt, uint32_t hpb, bool vec) {
    return ((size_t)qt * hpb * 2u * D + (size_t)kPage * diff_attn_ldk(ngk * 2u * D, vec) + (size_t)kPage * ngk * VD) * 4;
}
template <int VCH>
__device__ __forceinline__ void diff_finish(const DiffAttnArgs &a, const float (&o1)[VCH], const float (&o2)[VCH], float inv1, float inv2, size_t t, uint32_t h, uint32_t lane) {
    float dv[VCH], ss = 0.0f;
#pragma unroll
    for (int c = 0; c < VCH; c++) {
        const uint32_t r = lane + 32u * c;
        dv[c] = r < a.VD ? fmaf(-a.lambda, o2[c] * inv2, o1[c] * inv1) : 0.0f;
        ss = fmaf(dv[c], dv[c], ss);
    }
    ss = warp_sum(ss);
    const float f = a.out_scale / sqrtf(ss / (float)a.VD + a.eps);
#pragma unroll
    for (int c = 0; c < VCH; c++) { const uint32_t r = lane + 32u * c; if (r < a.VD) a.out[(t * a.H + h) * a.VD + r] = dv[c] * f; }
}
template <int VCH, int QT>
__global__ void __launch_bounds__(256, QT > 1 && VCH <= 4 ? 2 : 1) k_diff_attn(const DiffAttnArgs a) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const uint32_t hpb = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t H = a.H, D = a.D, D2 = 2u * D, VD = a.VD, rep = H / a.G;
    // the last query tile sees the most keys: tiles are handed out from the end, so the longest blocks start first
    const uint32_t tq0 = (gridDim.x - 1u - blockIdx.x) * QT, nq = min((uint32_t)QT, a.T - tq0), split = blockIdx.y, h0 = blockIdx.z * hpb, h = h0 + warp;
    const uint32_t g_lo = h0 / rep, ng = (min(H, h0 + hpb) - 1u) / rep - g_lo + 1u;
    const bool vec = diff_attn_vec(D, VD, a.ldq);
    const uint32_t KW = ng * D2, VW = ng * VD, LDK = diff_attn_ldk(a.ngk * D2, vec), LDV = a.ngk * VD;
    float *q_s = sm;                               // [QT][hpb][2 D], already times scale
    float *k_s = q_s + QT * hpb * D2;              // [kPage][LDK]
    float *v_s = k_s + kPage * LDK;                // [kPage][LDV]
    const uint32_t pos = a.pos0 + (a.pos_ptr ? *a.pos_ptr : 0u);
    const uint32_t nkeys = pos + tq0 + nq, tiles = (nkeys + kPage - 1u) / kPage;      // keys of the block's last query
    const uint32_t tps = (tiles + a.nsplit - 1u) / a.nsplit;
    const uint32_t tile_lo = split * tps, tile_hi = min(tiles, tile_lo + tps);
    for (uint32_t i = threadIdx.x; i < QT * hpb * D2; i += blockDim.x) {
        const uint32_t qi = i / (hpb * D2), rem = i % (hpb * D2), hh = h0 + rem / D2;
        q_s[i] = (qi < nq && hh < H) ? a.q[(size_t)(tq0 + qi) * a.ldq + hh * D2 + rem % D2] * a.scale : 0.0f;
    }
    float m[2][QT], l[2][QT], o[2][QT][VCH];
#pragma unroll
    for (int mp = 0; mp < 2; mp++)
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            m[mp][qi] = -INFINITY; l[mp][qi] = 0.0f;
#pragma unroll
            for (int c = 0; c < VCH; c++) o[mp][qi][c] = 0.0f;
        }
    const uint32_t g = (h < H ? h / rep : g_lo) - g_lo;
    for (uint32_t tile = tile_lo; tile < tile_hi; tile++) {
        __syncthreads();
        const float *src = a.cache + (size_t)a.table[tile] * kPage * a.RL;
        const uint32_t nk = min(kPage, nkeys - tile * kPage);
        const float *ksrc = src + g_lo * D2, *vsrc = src + a.G * D2 + g_lo * VD;
        if (vec) {
            // keys and values of the tile as one list of 16-byte pieces; a thread of a short portion's block (few warps, nothing else to
            // hide the latency behind) has eight of them in flight at once, a prefill block two (registers: two blocks per SM)
            constexpr int NB = QT == 1 ? 8 : 2;
            const uint32_t kw4 = KW / 4u, vw4 = VW / 4u, nk4 = nk * kw4, n4 = nk4 + nk * vw4;
            for (uint32_t base = 0; base < n4; base += NB * blockDim.x) {
                float4 v[NB];
#pragma unroll
                for (int k = 0; k < NB; k++) {
                    const uint32_t i = base + k * blockDim.x + threadIdx.x;
                    if (i < nk4) v[k] = __ldg(reinterpret_cast<const float4 *>(ksrc + (size_t)(i / kw4) * a.RL) + i % kw4);
                    else if (i < n4) v[k] = __ldg(reinterpret_cast<const float4 *>(vsrc + (size_t)((i - nk4) / vw4) * a.RL) + (i - nk4) % vw4);
                }
#pragma unroll
                for (int k = 0; k < NB; k++) {
                    const uint32_t i = base + k * blockDim.x + threadIdx.x;
                    if (i < nk4) *reinterpret_cast<float4 *>(k_s + (i / kw4) * LDK + (i % kw4) * 4u) = v[k];
                    else if (i < n4) *reinterpret_cast<float4 *>(v_s + ((i - nk4) / vw4) * LDV + ((i - nk4) % vw4) * 4u) = v[k];
                }
            }
        } else {
            for (uint32_t i = threadIdx.x; i < nk * KW; i += blockDim.x) k_s[(i / KW) * LDK + i % KW] = ksrc[(size_t)(i / KW) * a.RL + i % KW];
            for (uint32_t i = threadIdx.x; i < nk * VW; i += blockDim.x) v_s[(i / VW) * LDV + i % VW] = vsrc[(size_t)(i / VW) * a.RL + i % VW];
        }
        __syncthreads();
        if (h >= H) continue;
        uint32_t nkq[QT], nkmax = 0;               // keys of this tile each query sees (0: the tile lies after the query)
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            const uint32_t kq = pos + tq0 + qi + 1u;
            nkq[qi] = ((uint32_t)qi < nq && kq > tile * kPage) ? min(nk, kq - tile * kPage) : 0u;
            nkmax = max(nkmax, nkq[qi]);
        }
        float p[2][QT];
        const float *kr = k_s + lane * LDK + g * D2;         // lanes past nk read stale rows: their scores are selected away below
#pragma unroll
        for (int mp = 0; mp < 2; mp++) {
            float sc[QT];
#pragma unroll
            for (int qi = 0; qi < QT; qi++) sc[qi] = 0.0f;
            if (vec) {
                const float4 *k4 = reinterpret_cast<const float4 *>(kr + mp * D);
                for (uint32_t r4 = 0; r4 < D / 4u; r4++) {
                    const float4 kv = k4[r4];
#pragma unroll
                    for (int qi = 0; qi < QT; qi++) {
                        const float4 qv = reinterpret_cast<const float4 *>(q_s + ((size_t)qi * hpb + warp) * D2 + mp * D)[r4];
                        sc[qi] = fmaf(qv.w, kv.w, fmaf(qv.z, kv.z, fmaf(qv.y, kv.y, fmaf(qv.x, kv.x, sc[qi]))));
                    }
                }
            } else {
                for (uint32_t r = 0; r < D; r++) {
                    const float kv = kr[mp * D + r];
#pragma unroll
                    for (int qi = 0; qi < QT; qi++) sc[qi] = fmaf(q_s[((size_t)qi * hpb + warp) * D2 + mp * D + r], kv, sc[qi]);
                }
            }
#pragma unroll
            for (int qi = 0; qi < QT; qi++) {
                const bool seen = lane < nkq[qi];
                const float s = seen ? sc[qi] : -INFINITY;
                float tm = s;
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, off));
                const float mn = fmaxf(m[mp][qi], tm);
                const float corr = mn == -INFINITY ? 1.0f : expf(m[mp][qi] - mn);
                p[mp][qi] = seen ? expf(s - mn) : 0.0f;
                l[mp][qi] = l[mp][qi] * corr + warp_sum(p[mp][qi]);
                m[mp][qi] = mn;
#pragma unroll
                for (int c = 0; c < VCH; c++) o[mp][qi][c] *= corr;
            }
        }
        for (uint32_t j = 0; j < nkmax; j++) {
            float pj[2][QT];
#pragma unroll
            for (int mp = 0; mp < 2; mp++)
#pragma unroll
                for (int qi = 0; qi < QT; qi++) pj[mp][qi] = __shfl_sync(0xffffffffu, p[mp][qi], j);
            const float *vj = v_s + j * LDV + g * VD;
#pragma unroll
            for (int c = 0; c < VCH; c++) {
                const uint32_t r = lane + 32u * c;
                if (r < VD) {
                    const float vv = vj[r];
#pragma unroll
                    for (int qi = 0; qi < QT; qi++) { o[0][qi][c] = fmaf(pj[0][qi], vv, o[0][qi][c]); o[1][qi][c] = fmaf(pj[1][qi], vv, o[1][qi][c]); }
                }
            }
        }
    }
    if (a.nsplit == 1) {
        if (h >= H) return;
#pragma unroll
        for (int qi = 0; qi < QT; qi++)
            if ((uint32_t)qi < nq) diff_finish<VCH>(a, o[0][qi], o[1][qi], 1.0f / l[0][qi], 1.0f / l[1][qi], tq0 + qi, h, lane);
        return;
    }
    // key splits: partial triples of both maps, then the block that draws the last ticket merges,
    //   a_m = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s   over the splits that saw keys
    const uint32_t PW = VD + 2u;
    if (h < H) {
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            if ((uint32_t)qi >= nq) continue;
#pragma unroll
            for (int mp = 0; mp < 2; mp++) {
                float *dst = a.part + ((((size_t)(tq0 + qi) * a.nsplit + split) * H + h) * 2u + mp) * PW;
#pragma unroll
                for (int c = 0; c < VCH; c++) { const uint32_t r = lane + 32u * c; if (r < VD) dst[r] = o[mp][qi][c]; }
                if (lane == 0) { dst[VD] = m[mp][qi]; dst[VD + 1u] = l[mp][qi]; }
            }
        }
    }
    __shared__ uint32_t last_s;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t *tk = a.tickets + blockIdx.x * gridDim.z + blockIdx.z;
        const uint32_t got = atomicAdd(tk, 1u);
        last_s = got + 1u == a.nsplit;
        if (last_s) *tk = 0u;              // ready for the next launch
    }
    __syncthreads();
    if (!last_s || h >= H) return;
    __threadfence();
    const size_t stride = (size_t)H * 2u * PW;
#pragma unroll
    for (int qi = 0; qi < QT; qi++) {
        if ((uint32_t)qi >= nq) continue;
        const size_t t = tq0 + qi;
        float acc[2][VCH], inv[2], w[2];
        const float *base = a.part + ((size_t)t * a.nsplit * H + h) * 2u * PW;
#pragma unroll
        for (int mp = 0; mp < 2; mp++) {
            const bool live = lane < a.nsplit;
            const float ls = live ? __ldcg(base + lane * stride + mp * PW + VD + 1u) : 0.0f;
            const float ms = (live && ls > 0.0f) ? __ldcg(base + lane * stride + mp * PW + VD) : -INFINITY;
            float M = ms;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
            w[mp] = ls > 0.0f ? expf(ms - M) : 0.0f;
            inv[mp] = 1.0f / warp_sum(w[mp] * ls);
#pragma unroll
            for (int c = 0; c < VCH; c++) acc[mp][c] = 0.0f;
        }
        // every split wrote its triples in this launch (zeros where it saw no key), so the loop needs no branch and its loads overlap
#pragma unroll 4
        for (uint32_t sp = 0; sp < a.nsplit; sp++) {
            const float w0 = __shfl_sync(0xffffffffu, w[0], sp), w1 = __shfl_sync(0xffffffffu, w[1], sp);
#pragma unroll
            for (int c = 0; c < VCH; c++) {
                const uint32_t r = lane + 32u * c;
                if (r < VD) { acc[0][c] = fmaf(w0, __ldcg(base + sp * stride + r), acc[0][c]); acc[1][c] = fmaf(w1, __ldcg(base + sp * stride + PW + r), acc[1][c]); }
            }
        }
        diff_finish<VCH>(a, acc[0], acc[1], inv[0], inv[1], t, h, lane);
    }
}

// Mamba-2 recurrence, token by token.  A block of 8 warps owns 8 x CPW value columns of head h = blockIdx.y (a warp CPW of them) and
// keeps S[h][j][:] in registers (lane l holds state coordinates l, l + 32, ...).  Per token, with dt = softplus(raw + dt_bias[h]) and
// a = exp(-rate[h] dt):   S[j][n] <- a S[j][n] + (dt x_j) B_n,   y_j = sum_n S[j][n] C_n + D[h] x_j.
// x, B and C come from the rows of xbc (the convolved, activated [x | B | C]): x at column h P, B at Hn P + g N, C at Hn P + (G + g) N
// with g = h / (Hn / G); 32 (or 16) tokens at a time are staged in shared memory.  The decay is made in double precision and rounded
// once: a state that forgets slowly takes thousands of these steps, and an error of the decay beyond its own rounding would
// accumulate over them.  State [Hn][P][N] fp32; y [T][Hn P].
// Long portions run parallel over time (gridDim.z segments of seg_len tokens): mode 1 builds every segment's state from zero into
// seg_S[segment] (no outputs), k_ssd_chain turns those into the states the segments start from (and the slot's state after the
// portion), mode 2 replays every segment from seg_S[segment] with outputs.  mode 0: one pass from and to S.
struct SsdArgs {
    const float *xbc; uint32_t ldx; const float *dt; uint32_t lddt; const float *dt_bias, *rate, *Dv;
    float *S; float *y; uint32_t T, Hn, P, N, G; uint32_t mode, seg_len; float *seg_S;
    const float *z; uint32_t ldz;      // the gate: what is written is y silu(z[t][h P + j])
};
__device__ __forceinline__ float ssd_decay(float rate, float dt) { return (float)exp(-(double)rate * (double)dt); }
template <int DCH, int CPW>
__global__ void __launch_bounds__(256) k_ssd_scan(const SsdArgs a) {
    pdl_enter();
    constexpr uint32_t kCols = 8 * CPW, kTile = DCH <= 4 ? 32 : 16;
    __shared__ float Bs[kTile][DCH * 32], Cs[kTile][DCH * 32], xs[kTile][kCols], xr[kTile][kCols], zs[kTile][kCols], as[kTile], ds[kTile];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, h = blockIdx.y, j0 = blockIdx.x * kCols, jw = j0 + warp * CPW;
    const uint32_t g = h / (a.Hn / a.G), xoff = h * a.P, boff = a.Hn * a.P + g * a.N, coff = a.Hn * a.P + (a.G + g) * a.N;
    float *Sio = a.mode ? a.seg_S + (size_t)blockIdx.z * a.Hn * a.P * a.N : a.S;
    const uint32_t t_lo = a.mode ? blockIdx.z * a.seg_len : 0u, t_hi = a.mode ? min(a.T, t_lo + a.seg_len) : a.T;
    float S[CPW][DCH];
#pragma unroll
    for (uint32_t i = 0; i < CPW; i++)
#pragma unroll
        for (int c = 0; c < DCH; c++) { const uint32_t n = lane + 32u * c; S[i][c] = (a.mode != 1u && jw + i < a.P && n < a.N) ? Sio[((size_t)h * a.P + jw + i) * a.N + n] : 0.0f; }
    const float rate = a.rate[h], bias = a.dt_bias[h], Dh = a.Dv[h];
    for (uint32_t t0 = t_lo; t0 < t_hi; t0 += kTile) {
        const uint32_t nt = min(kTile, t_hi - t0);
        __syncthreads();
        if (threadIdx.x < nt) {
            const float dt = softplusf_(a.dt[(size_t)(t0 + threadIdx.x) * a.lddt + h] + bias);
            ds[threadIdx.x] = dt; as[threadIdx.x] = ssd_decay(rate, dt);
        }
        for (uint32_t i = threadIdx.x; i < nt * DCH * 32u; i += blockDim.x) {
            const uint32_t t = i / (DCH * 32u), n = i % (DCH * 32u);
            const float *row = a.xbc + (size_t)(t0 + t) * a.ldx;
            Bs[t][n] = n < a.N ? row[boff + n] : 0.0f;
            Cs[t][n] = (n < a.N && a.mode != 1u) ? row[coff + n] : 0.0f;
        }
        __syncthreads();
        for (uint32_t i = threadIdx.x; i < nt * kCols; i += blockDim.x) {
            const uint32_t t = i / kCols, j = i % kCols;
            const float v = j0 + j < a.P ? a.xbc[(size_t)(t0 + t) * a.ldx + xoff + j0 + j] : 0.0f;
            xr[t][j] = v; xs[t][j] = v * ds[t];
            if (a.mode != 1u) zs[t][j] = j0 + j < a.P ? siluf_(a.z[(size_t)(t0 + t) * a.ldz + xoff + j0 + j]) : 0.0f;
        }
        __syncthreads();
        if (a.mode == 1u) {          // the first pass of a long portion only builds states
            for (uint32_t t = 0; t < nt; t++) {
                const float av = as[t];
                float v[CPW];
#pragma unroll
                for (uint32_t i = 0; i < CPW; i++) v[i] = xs[t][warp * CPW + i];
#pragma unroll
                for (int c = 0; c < DCH; c++) {
                    const float bn = Bs[t][lane + 32 * c];
#pragma unroll
                    for (uint32_t i = 0; i < CPW; i++) S[i][c] = fmaf(av, S[i][c], bn * v[i]);
                }
            }
            continue;
        }
        for (uint32_t t = 0; t < nt; t++) {
            const float av = as[t];
            float acc[CPW], v[CPW];
#pragma unroll
            for (uint32_t i = 0; i < CPW; i++) { acc[i] = 0.0f; v[i] = xs[t][warp * CPW + i]; }
#pragma unroll
            for (int c = 0; c < DCH; c++) {
                const float bn = Bs[t][lane + 32 * c], cn = Cs[t][lane + 32 * c];
#pragma unroll
                for (uint32_t i = 0; i < CPW; i++) { S[i][c] = fmaf(av, S[i][c], bn * v[i]); acc[i] = fmaf(S[i][c], cn, acc[i]); }
            }
            float *yrow = a.y + (size_t)(t0 + t) * a.Hn * a.P + xoff + jw;
            if (CPW == 4) {
                // four sums over the warp with six shuffles: halves of the warp trade two columns, quarters one, then eight lanes add up;
                // lanes 0, 8, 16, 24 end with columns 0, 1, 2, 3
                const bool h16 = lane & 16u, h8 = lane & 8u;
                float k0 = (h16 ? acc[2] : acc[0]) + __shfl_xor_sync(0xffffffffu, h16 ? acc[0] : acc[2], 16);
                float k1 = (h16 ? acc[3] : acc[1]) + __shfl_xor_sync(0xffffffffu, h16 ? acc[1] : acc[3], 16);
                float k = (h8 ? k1 : k0) + __shfl_xor_sync(0xffffffffu, h8 ? k0 : k1, 8);
                k += __shfl_xor_sync(0xffffffffu, k, 4); k += __shfl_xor_sync(0xffffffffu, k, 2); k += __shfl_xor_sync(0xffffffffu, k, 1);
                const uint32_t col = lane >> 3;
                if ((lane & 7u) == 0 && jw + col < a.P) yrow[col] = fmaf(Dh, xr[t][warp * CPW + col], k) * zs[t][warp * CPW + col];
            } else {
#pragma unroll
                for (uint32_t i = 0; i < CPW; i++) acc[i] = warp_sum(acc[i]);
                float mine = acc[0];
#pragma unroll
                for (uint32_t i = 1; i < CPW; i++) if (lane == i) mine = acc[i];
                if (lane < CPW && jw + lane < a.P) yrow[lane] = fmaf(Dh, xr[t][warp * CPW + lane], mine) * zs[t][warp * CPW + lane];
            }
        }
    }
    if (a.mode == 2u) return;
#pragma unroll
    for (uint32_t i = 0; i < CPW; i++)
#pragma unroll
        for (int c = 0; c < DCH; c++) { const uint32_t n = lane + 32u * c; if (jw + i < a.P && n < a.N) Sio[((size_t)h * a.P + jw + i) * a.N + n] = S[i][c]; }
}

// Between the two passes of a long portion: seg_S[s] holds what segment s built from zero; it becomes the state segment s starts
// from, S_s = A_(s-1) S_(s-1) + built(s-1) with A_s = exp(-rate sum of the segment's dt), S_0 = the slot's state, which in turn
// becomes the state after the last segment.  grid = (blocks over a head's state, heads); nseg <= 8 = the warps of a block.
struct SsdChainArgs { float *S; float *seg_S; const float *dt; uint32_t lddt; const float *dt_bias, *rate; uint32_t Hn, P, N, T, seg_len, nseg; };
__global__ void __launch_bounds__(256) k_ssd_chain(const SsdChainArgs a) {
    pdl_enter();
    __shared__ float dec[8];
    const uint32_t h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (warp < a.nseg) {
        const uint32_t t0 = warp * a.seg_len, t1 = min(a.T, t0 + a.seg_len);
        const float bias = a.dt_bias[h];
        double s = 0.0;
        for (uint32_t t = t0 + lane; t < t1; t += 32u) s += (double)softplusf_(a.dt[(size_t)t * a.lddt + h] + bias);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) dec[warp] = (float)exp(-(double)a.rate[h] * s);
    }
    __syncthreads();
    const uint32_t per = a.P * a.N;
    const size_t total = (size_t)per * a.Hn;
    for (uint32_t j = blockIdx.x * blockDim.x + threadIdx.x; j < per; j += gridDim.x * blockDim.x) {
        const size_t i = (size_t)h * per + j;
        float built[8];
#pragma unroll
        for (uint32_t sg = 0; sg < 8; sg++) built[sg] = sg < a.nseg ? a.seg_S[(size_t)sg * total + i] : 0.0f;
        float s = a.S[i];
#pragma unroll
        for (uint32_t sg = 0; sg < 8; sg++) {
            if (sg >= a.nseg) break;
            a.seg_S[(size_t)sg * total + i] = s;
            s = fmaf(dec[sg], s, built[sg]);
        }
        a.S[i] = s;
    }
}

// group norm and gain: every one of the `parts` equal parts of a token's row is divided by its own root mean square (eps inside the
// root) and multiplied by the gain.  One block per (token, part).  (Short portions: the prologue of the product that follows, GemmArgs::a_parts.)
struct GroupNormArgs { const float *y; const float *gain; float *out; uint32_t T, C, parts; float eps; };
__global__ void __launch_bounds__(1024) k_group_norm(const GroupNormArgs a) {
    pdl_enter();
    __shared__ float red[32];
    const uint32_t t = blockIdx.x / a.parts, part = blockIdx.x % a.parts, W = a.C / a.parts, c0 = part * W;
    const float *y = a.y + (size_t)t * a.C + c0;
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < W; i += blockDim.x) s = fmaf(y[i], y[i], s);
    s = block_sum(s, red);
    const float rinv = 1.0f / sqrtf(s / (float)W + a.eps);
    float *out = a.out + (size_t)t * a.C + c0;
    for (uint32_t i = threadIdx.x; i < W; i += blockDim.x) out[i] = y[i] * rinv * a.gain[c0 + i];
}

}  // namespace lm
}  // namespace nb

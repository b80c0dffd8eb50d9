// layered_mixers3.cuh -- more mechanisms of the layered runtime (layered.cu), each with its constants as arguments:
//
//   hyper-connections    k_hc_step: the residual is S streams.  After a sublayer,  x_t <- sum_s mix[s][t] x_s + mult * out[t] * ls * y
//                        (all streams at once from the old ones; ls a per-channel layer scale, y the sublayer's output or the weighted
//                        sum of the chosen experts' rows plus a shared expert), and in the same pass the NEXT sublayer's input: the
//                        bias-free layer norm of  u = sum_s in[s] x_s.  One stream with mix = in = out = 1 is the plain pre-norm
//                        residual  x += mult * ls * y.  The first step of a portion fills the streams from the embedding table
//                        (token row times a fixed scale, copied into every stream).  k_final_ln: layer norm of the sum of the streams.
//   latent + rotated key k_latent_rope: the key/value latent of a token (first R columns of its down-projection, RMS-normed with a vector
//                        gain) and, beside it, a rotated key part shared by all heads (the next RD columns, pairs (2i, 2i+1) turned by
//                        position x frequency) go into the token's cache row [R | RD | padding]; the rotated part of every head's
//                        query goes to the same columns of the head's absorbed-query row, so that k_latent_attn scores
//                        q_latent . c + q_rot . k_rot with one dot product.  k_gemv_latent_rope: the same rows done by one block of the
//                        absorb product of a short portion.
#pragma once
#include "layered_mixers2.cuh"

namespace nb {
namespace lm {

constexpr uint32_t kMaxStreams = 8;

// hc: the sublayer's connection weights [in S | out S | mix S x S (from, to)]; next_in: the `in` weights of the sublayer that follows
struct HcArgs {
    float *xs; size_t s_stride; uint32_t S;                     // stream s of token t: xs + s * s_stride + t * E
    const float *y;                                             // the sublayer's output [T][E] (null with eo, or in the first step)
    const float *eo; const uint32_t *slot; const float *wt; uint32_t top; const float *shared;      // experts' rows instead of y
    const float *ls; const float *hc; float mult;
    const float *next_in, *next_w; float *out;                  // the next sublayer's input norm (out null: no sublayer follows)
    float *keep;                                                // optional: the sum of the streams
    uint32_t T, E; float eps;
    const uint32_t *tokens; const uint32_t *pos_ptr; const void *embed; float emb_scale;      // first step: streams <- embed[token] * scale
};
// SC: a compile-time bound of the stream count (1, 2, 4 or kMaxStreams), so that the small loops over the streams unroll to their size
template <typename WT, int SC>
__global__ void __launch_bounds__(1024) k_hc_step(const HcArgs a) {
    pdl_enter();
    __shared__ float red[32];
    __shared__ float w_in[kMaxStreams], w_out[kMaxStreams], w_mix[kMaxStreams * kMaxStreams];
    const uint32_t t = blockIdx.x, S = a.S, E = a.E;
    if (threadIdx.x < S) {
        w_in[threadIdx.x] = a.next_in ? a.next_in[threadIdx.x] : 0.0f;
        w_out[threadIdx.x] = a.hc ? a.hc[S + threadIdx.x] * a.mult : 0.0f;
    }
    if (threadIdx.x < S * S) w_mix[threadIdx.x] = a.hc ? a.hc[2u * S + threadIdx.x] : 0.0f;
    __syncthreads();
    const WT *erow = a.tokens ? static_cast<const WT *>(a.embed) + (size_t)a.tokens[t + (a.pos_ptr ? *a.pos_ptr : 0u)] * E : nullptr;
    float *x0 = a.xs + (size_t)t * E;
    float *orow = a.out ? a.out + (size_t)t * E : nullptr;
    float sum = 0.0f;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) {
        float nx[SC];
        if (erow) {
            const float v = wval(erow + i) * a.emb_scale;
#pragma unroll
            for (uint32_t s = 0; s < (uint32_t)SC; s++) nx[s] = v;
        } else {
            float y;
            if (a.eo) {
                y = 0.0f;
                for (uint32_t j = 0; j < a.top; j++) y = fmaf(a.wt[(size_t)t * a.top + j], a.eo[(size_t)a.slot[(size_t)t * a.top + j] * E + i], y);
                if (a.shared) y += a.shared[(size_t)t * E + i];
            } else y = a.y[(size_t)t * E + i];
            if (a.ls) y *= a.ls[i];
            float old[SC];
#pragma unroll
            for (uint32_t s = 0; s < (uint32_t)SC; s++) old[s] = s < S ? x0[s * a.s_stride + i] : 0.0f;
#pragma unroll
            for (uint32_t r = 0; r < (uint32_t)SC; r++) {
                float v = 0.0f;
                if (r < S) {
#pragma unroll
                    for (uint32_t s = 0; s < (uint32_t)SC; s++) if (s < S) v = fmaf(w_mix[s * S + r], old[s], v);
                    v = fmaf(w_out[r], y, v);
                }
                nx[r] = v;
            }
        }
        float u = 0.0f, tot = 0.0f;
#pragma unroll
        for (uint32_t s = 0; s < (uint32_t)SC; s++)
            if (s < S) { x0[s * a.s_stride + i] = nx[s]; u = fmaf(w_in[s], nx[s], u); tot += nx[s]; }
        if (a.keep) a.keep[(size_t)t * E + i] = tot;
        if (orow) { orow[i] = u; sum += u; }
    }
    if (!orow) return;
    // bias-free layer norm of u, in three passes over the thread's own elements: mean, mean of the squared deviations, the result
    const float mean = block_sum(sum, red) / (float)E;
    float sq = 0.0f;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) { const float c = orow[i] - mean; sq = fmaf(c, c, sq); }
    const float rstd = 1.0f / sqrtf(block_sum(sq, red) / (float)E + a.eps);
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) orow[i] = (orow[i] - mean) * rstd * a.next_w[i];
}

// out[r] = layer norm (gain w, no bias) of the sum of the streams of row want[r]
__global__ void __launch_bounds__(1024) k_final_ln(const float *__restrict__ xs, size_t s_stride, uint32_t S, const uint32_t *__restrict__ want,
                                                  const float *__restrict__ w, float *__restrict__ out, uint32_t E, float eps) {
    pdl_enter();
    __shared__ float red[32];
    const float *x0 = xs + (size_t)want[blockIdx.x] * E;
    float *orow = out + (size_t)blockIdx.x * E;
    float sum = 0.0f;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) {
        float v = 0.0f;
        for (uint32_t s = 0; s < S; s++) v += x0[s * s_stride + i];
        orow[i] = v; sum += v;
    }
    const float mean = block_sum(sum, red) / (float)E;
    float sq = 0.0f;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) { const float c = orow[i] - mean; sq = fmaf(c, c, sq); }
    const float rstd = 1.0f / sqrtf(block_sum(sq, red) / (float)E + eps);
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) orow[i] = (orow[i] - mean) * rstd * w[i];
}

// z rows: every head's query [H][D + RD] at column q0, the down-projection [R + RD] at column z0.  tab[position][i] = (cos, sin) of
// position x f_i for i < dims / 2 (dims <= RD; coordinates past dims pass unchanged).  qa rows: [H][RS], RS >= R + RD.
struct LatentRopeArgs {
    const float *z; uint32_t ldz, q0, z0; const float *wkv; float *cache; const uint32_t *table; float *qa;
    uint32_t T, H, D, RD, R, RS, dims; const float2 *tab; uint32_t pos0; float eps; const uint32_t *pos_ptr;
};
// one value of the rotated part `src` [RD] at coordinate i
__device__ __forceinline__ float rot_coord(const float *src, uint32_t i, uint32_t dims, const float2 *tab_row) {
    if (i >= dims) return src[i];
    const float2 cs = tab_row[i >> 1];
    return (i & 1u) ? fmaf(src[i], cs.x, src[i - 1u] * cs.y) : fmaf(src[i], cs.x, -src[i + 1u] * cs.y);
}
__device__ __forceinline__ void latent_rope_row(const LatentRopeArgs &a, uint32_t t, float *red) {
    const float *z = a.z + (size_t)t * a.ldz + a.z0;
    float s2 = 0.0f;
    for (uint32_t i = threadIdx.x; i < a.R; i += blockDim.x) s2 = fmaf(z[i], z[i], s2);
    s2 = block_sum(s2, red);
    const float rk = 1.0f / sqrtf(s2 / (float)a.R + a.eps);
    const uint32_t pos = a.pos0 + t + (a.pos_ptr ? *a.pos_ptr : 0u);
    float *row = a.cache + ((size_t)a.table[pos / kPage] * kPage + pos % kPage) * a.RS;
    const float2 *tab_row = a.tab ? a.tab + (size_t)pos * (a.dims / 2u) : nullptr;
    const uint32_t dims = a.tab ? a.dims : 0u, X = a.RS - a.R;
    for (uint32_t i = threadIdx.x; i < a.R; i += blockDim.x) row[i] = z[i] * rk * a.wkv[i];
    for (uint32_t i = threadIdx.x; i < X; i += blockDim.x) row[a.R + i] = i < a.RD ? rot_coord(z + a.R, i, dims, tab_row) : 0.0f;
    for (uint32_t j = threadIdx.x; j < a.H * X; j += blockDim.x) {
        const uint32_t h = j / X, i = j % X;
        const float *q = a.z + (size_t)t * a.ldz + a.q0 + (size_t)h * (a.D + a.RD) + a.D;
        a.qa[((size_t)t * a.H + h) * a.RS + a.R + i] = i < a.RD ? rot_coord(q, i, dims, tab_row) : 0.0f;
    }
}
__global__ void __launch_bounds__(128) k_latent_rope(const LatentRopeArgs a) {
    pdl_enter();
    __shared__ float red[32];
    latent_rope_row(a, blockIdx.x, red);
}
// Short portions: the last block of the absorb product (a grouped product, one group per head) also norms, turns and caches.
struct GemvLatentRopeArgs { GemmArgs g; LatentRopeArgs n; };
template <typename WT>
__global__ void __launch_bounds__(256) k_gemv_latent_rope(const GemvLatentRopeArgs a) {
    pdl_launch_next();
    gemv_prefetch<WT>(a.g);
    pdl_wait();
    __shared__ float red[32];
    if (blockIdx.x == gridDim.x - 1u && blockIdx.y == gridDim.y - 1u)
        for (uint32_t t = 0; t < a.n.T; t++) latent_rope_row(a.n, t, red);
    gemv_body<WT>(a.g, red);
}

}  // namespace lm
}  // namespace nb

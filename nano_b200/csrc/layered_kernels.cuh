// layered_kernels.cuh -- device code of the layered runtime (layered.cu): models that are a list of typed layers, each a token
// mixer plus an optional feed-forward, over an fp32 residual stream.  Every mechanism is a kernel (or a GEMM epilogue) of its own
// with its constants as arguments, so a new design combines them by configuration:
//
//   matrix products      k_gemm_f32 (fp32 FMA tiles, the true-32-bit mode), k_gemm_bf16 (mma.sync m16n8k16, bf16 operands, fp32
//                        accumulators: prefill), k_gemv (a warp per output row, weights streamed once: decode and portions of <= 4 tokens).
//                        One argument block serves plain, grouped (block-diagonal gates, per-head absorb / value up-projection) and
//                        routed (rows gathered per expert, group sizes read on the device) products; bias / gelu_tanh / sigmoid /
//                        squared-relu epilogues.
//   norms                k_norm_shift (RMS norm with ONE scalar gain, two gains of the same x at once, + token shift of the mixer's
//                        input against the previous token's input, carried in the sequence state), k_latent_norm (vector-gain RMS norm
//                        of the query latent and of the key/value latent, the latter written into the paged cache; for short portions
//                        k_gemv_latent does both inside the query up-projection), k_final_norm
//   recurrence           k_conv / k_conv_state (causal per-channel convolution with its taps-1 tail in the state; for short portions it is
//                        an epilogue of k_gemv), k_rglru_scan (real-gated linear recurrent unit: a = exp(-c r softplus(lam)),
//                        S = a S + sqrt(1 - a^2) i u, fp32 state; token by token), k_rglru_scan_par (the same, parallel over time
//                        segments, for long portions) and k_rglru_gates_scan (both gate products + the recurrence, short portions)
//   attention            k_latent_attn (softmax attention of absorbed queries directly over cached latents: the latent is key AND
//                        value, positions-free, causal; split over the keys for decode, merged by the block that finishes last)
//   mixture of experts   k_route (fp32 router logits -> top-k, softmax over the chosen), k_route_place (expert-sorted slots), k_route_small
//                        (both in one block, short portions),
//                        k_combine (weighted sum in choice order + shared expert + mixer output -> residual)
//
// More mechanisms (position table, sandwich norms, rotary positions, retention, window attention, selective scan, PolyNorm) live in
// layered_mixers.cuh under the same rules.
//
// What is fp32 here regardless of the weight type: the residual stream, every norm, router logits, attention scores / weights /
// accumulators, gates, decays and the recurrent state.  bf16 enters only as a matrix-product operand.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace nb {
namespace lm {

constexpr uint32_t kPage = 32;            // tokens per cache page == keys per attention tile
constexpr uint32_t kAttnWarps = 8;        // heads per attention block
constexpr uint32_t kGemvMaxM = 4;         // rows a k_gemv launch handles per group

enum CMode : uint32_t { C_ADD = 1, C_SCALE = 2 };
enum Epi : uint32_t { EPI_NONE = 0, EPI_BIAS = 1, EPI_GELU_SPLIT = 2, EPI_SIGMOID = 3, EPI_RELU2 = 4, EPI_GELU_CONV = 5, EPI_SOFTPLUS = 6, EPI_CONV_RANGES = 7, EPI_SIGMOID_TAIL = 8, EPI_GELU_ERF = 9 };

// C[r, c0 + n] = epi( sum_k A[arow(r), a0 + k] * W[g][n, k] + bias[g][n] )   for the rows r of group g
//   rows of group g : [g_off[g], g_off[g+1])  when g_off is given (sizes known on the device only), else [0, M)
//   arow(r)         : a_rows[r] when given (gather), else r
//   a0 = (g % a_gmod) * a_gcols,  c0 = g * c_gcols,  W[g] = W + g * w_gstride,  bias[g] = bias + g * b_gstride
struct GemmArgs {
    const float *A; const void *W; float *C; const float *bias;
    const uint32_t *g_off; const uint32_t *a_rows;
    uint32_t M, N, K, lda, ldw, ldc;
    uint32_t a_gmod, a_gcols, c_gcols, b_gstride;
    uint64_t w_gstride;
    uint32_t epi, split;      // EPI_GELU_SPLIT: gelu_tanh on columns n < split, bias only on the others; EPI_SIGMOID_TAIL: sigmoid on columns n >= split
    uint32_t round_a;         // k_gemv: round A to bf16 first (what the tensor-core kernel does to its operand)
    // k_gemv only.  Prologue: when a_norm_w is given, row r of A is used as A[r, k] / rms(A[r, 0..K)) * a_norm_w[k] (eps inside the root).
    const float *a_norm_w; float a_eps;
    // k_gemv only.  Epilogue EPI_GELU_CONV: columns n < split get gelu_tanh and go to C; a column n >= split is channel c = n - split of a
    // causal convolution over the rows in order (taps cv_taps[c][cv_K], bias cv_bias, tail cv_state [cv_K - 1][N - split]) whose
    // outputs go to cv_out [rows][N - split]; the tail moves on.  One warp owns a channel, so the tail has one reader and one writer.
    const float *cv_taps, *cv_bias; float *cv_state, *cv_out; uint32_t cv_K;
    // After the epilogue: with c_mode & C_SCALE the value is multiplied by c_scale, with c_mode & C_ADD it is added to what C holds,
    // so two products can be summed with fixed weights into one output (C = s1 A1 W1^T, then C += s2 A2 W2^T).
    float c_scale; uint32_t c_mode;
    // k_gemv only.  Prologue: when a_poly is given (4 numbers a, b, c, e), row r of A is used as a N(z) + b N(z^2) + c N(z^3) + e with
    // z = A[r, 0..K), powers element by element and N(u) = u / sqrt(mean(u^2) + a_eps).
    const float *a_poly;
    // k_gemv only.  Epilogue EPI_CONV_RANGES: a column n inside [cr[i].n0, cr[i].n1) is channel n - n0 of causal convolution i over the
    // rows in order (no epilogue before it); every other column is stored as usual.
    struct ConvRange { uint32_t n0, n1; const float *taps, *bias; float *state, *out; uint32_t K, act; } cr[2];
    // k_gemv only.  Gated pair (glu 1: gelu_tanh, 2: silu, 3: the clamped unit below): W holds 2 N rows per group, [gate rows | up rows]; column n of C receives
    // act(s g_n) (s u_n) with g_n, u_n the products of rows n and N + n and s = row_scale[row] (1 when null): a routed expert whose
    // input is weighted by the router's score, without a pass over the input.
    uint32_t glu; const float *row_scale;
    // k_gemv only.  Prologue (with a_norm_w): a_parts > 1 norms row r of A in a_parts equal parts, each by its own root mean square
    // (K / a_parts columns each, a multiple of 8; at most 32 parts).
    uint32_t a_parts;
    // k_gemv only (instances EXT 4 and 5).  Residual epilogue of a sublayer's last product, for designs whose norms are elementwise
    // (Dynamic Tanh, tanh(alpha u) w + b): instead of storing C, column n of row r updates the residual stream in place,
    // x[r][n] += tanh(res_pa v) res_pw[n] + res_pb[n], keeps a copy (res_keep, optional) and writes the next sublayer's input
    // res_out[r][n] = tanh(res_na x[r][n]) res_nw[n] + res_nb[n] (res_out optional).  Rows of x, res_out and res_keep are N long.
    float *res_x, *res_out, *res_keep; const float *res_pw, *res_pb, *res_nw, *res_nb; float res_pa, res_na;
    // After the epilogue: with mul given, the value of row r (of the output) and column c0 + n is multiplied by mul[r * ldm + c0 + n]
    // (an output gate computed by an earlier product).
    const float *mul; uint32_t ldm;
    // Gated pair, glu 3: the clamped unit  g' = min(g, glu_limit), u' = clamp(u, -glu_limit, glu_limit),  g' sigmoid(1.702 g') (u' + 1).
    float glu_limit;
};

// Programmatic dependent launch: every kernel first lets the NEXT kernel of its stream be scheduled (its blocks then sit in their own
// pdl_enter until this grid has finished and its writes are visible), then waits for the kernels before it.  Launch latency and block
// scheduling of a chain of short kernels overlap with the tail of the kernel before; no kernel reads or writes what another kernel
// produces before the wait (weights may be prefetched: nothing writes them).
__device__ __forceinline__ void pdl_launch_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_enter() { pdl_launch_next(); pdl_wait(); }
// Weights do not depend on the kernel before: a matrix-vector kernel asks for its weight rows (L2 prefetch, no register, no wait)
// BETWEEN the two halves of pdl_enter, so their trip from HBM overlaps the tail of the kernel it waits for.  One 128-byte line per
// lane and step; at most `cols` rows per warp.
__device__ __forceinline__ void prefetch_weight_rows(const void *W, size_t elem, uint32_t ldw, uint32_t K, uint32_t N, uint32_t warp0, uint32_t nwarps, uint32_t cols) {
    const uint32_t lane = threadIdx.x & 31u, row_bytes = K * (uint32_t)elem;
    for (uint32_t n = warp0, c = 0; n < N && c < cols; n += nwarps, c++) {
        const char *p = static_cast<const char *>(W) + (size_t)n * ldw * elem;
        for (uint32_t off = lane * 128u; off < row_bytes; off += 32u * 128u) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + off));
    }
}

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.0f); }
// the clamped gated unit: the gate is capped from above, the linear branch on both sides and shifted by one
__device__ __forceinline__ float clamped_glu(float g, float u, float limit) {
    g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit);
    return g * sigmoidf_(1.702f * g) * (u + 1.0f);
}

__device__ __forceinline__ float epilogue(float v, const GemmArgs &a, const float *bias, uint32_t n) {
    if (bias) v += bias[n];
    switch (a.epi) {
        case EPI_GELU_SPLIT: case EPI_GELU_CONV: return n < a.split ? gelu_tanh(v) : v;
        case EPI_SIGMOID: return sigmoidf_(v);
        case EPI_RELU2: { const float r = fmaxf(v, 0.0f); return r * r; }
        case EPI_SOFTPLUS: return softplusf_(v);
        case EPI_SIGMOID_TAIL: return n >= a.split ? sigmoidf_(v) : v;
        case EPI_GELU_ERF: return 0.5f * v * (1.0f + erff(v * 0.70710678118654752f));
        default: return v;
    }
}
__device__ __forceinline__ float gated(const GemmArgs &a, float v, uint32_t row, uint32_t col) { return a.mul ? v * a.mul[(size_t)row * a.ldm + col] : v; }
__device__ __forceinline__ void store_c(const GemmArgs &a, float *dst, float v) {
    if (a.c_mode & C_SCALE) v *= a.c_scale;
    *dst = (a.c_mode & C_ADD) ? *dst + v : v;
}

struct GroupView { uint32_t r0, rows, a0, c0; const float *bias; uint64_t w0; };
__device__ __forceinline__ GroupView group_view(const GemmArgs &a, uint32_t g) {
    GroupView v;
    v.r0 = a.g_off ? a.g_off[g] : 0u;
    v.rows = a.g_off ? a.g_off[g + 1] - v.r0 : a.M;
    v.a0 = (g % a.a_gmod) * a.a_gcols; v.c0 = g * a.c_gcols;
    v.bias = a.bias ? a.bias + (size_t)g * a.b_gstride : nullptr;
    v.w0 = (uint64_t)g * a.w_gstride;
    return v;
}

__device__ __forceinline__ float wval(const float *w) { return *w; }
__device__ __forceinline__ float wval(const __nv_bfloat16 *w) { return __bfloat162float(*w); }

// ------------------------------------------------------------------------------------------------
// fp32 tile product: 64 x 64 output tile, 16-deep k steps, 256 threads with a 4 x 4 micro-tile each; plain FMA in k order
// ------------------------------------------------------------------------------------------------
template <typename WT>
__global__ void __launch_bounds__(256) k_gemm_f32(const GemmArgs a) {
    pdl_enter();
    const GroupView gv = group_view(a, blockIdx.z);
    const uint32_t m0 = blockIdx.y * 64u, n0 = blockIdx.x * 64u;
    if (m0 >= gv.rows) return;
    __shared__ float As[16][64 + 4], Bs[16][64 + 4];
    __shared__ uint32_t arow[64];
    const uint32_t tid = threadIdx.x, ty = tid >> 4, tx = tid & 15u;
    if (tid < 64) {
        const uint32_t r = m0 + tid;
        arow[tid] = r < gv.rows ? (a.a_rows ? a.a_rows[gv.r0 + r] : gv.r0 + r) : 0xffffffffu;
    }
    __syncthreads();
    const WT *W = static_cast<const WT *>(a.W) + gv.w0;
    float acc[4][4] = {};
    const uint32_t lr = tid >> 2, lk = (tid & 3u) * 4u;       // this thread stages 4 consecutive k of one row, for A and for W
    for (uint32_t k0 = 0; k0 < a.K; k0 += 16u) {
        {
            const uint32_t ar = arow[lr];
            const float *src = a.A + (size_t)ar * a.lda + gv.a0 + k0 + lk;
#pragma unroll
            for (uint32_t j = 0; j < 4; j++) As[lk + j][lr] = (ar != 0xffffffffu && k0 + lk + j < a.K) ? src[j] : 0.0f;
            const uint32_t n = n0 + lr;
            const WT *ws = W + (size_t)n * a.ldw + k0 + lk;
#pragma unroll
            for (uint32_t j = 0; j < 4; j++) Bs[lk + j][lr] = (n < a.N && k0 + lk + j < a.K) ? wval(ws + j) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (uint32_t k = 0; k < 16; k++) {
            float av[4], bv[4];
#pragma unroll
            for (uint32_t i = 0; i < 4; i++) { av[i] = As[k][ty * 4 + i]; bv[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
            for (uint32_t i = 0; i < 4; i++)
#pragma unroll
                for (uint32_t j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (uint32_t i = 0; i < 4; i++) {
        const uint32_t r = m0 + ty * 4 + i;
        if (r >= gv.rows) continue;
#pragma unroll
        for (uint32_t j = 0; j < 4; j++) {
            const uint32_t n = n0 + tx * 4 + j;
            if (n < a.N) store_c(a, a.C + (size_t)(gv.r0 + r) * a.ldc + gv.c0 + n, gated(a, epilogue(acc[i][j], a, gv.bias, n), gv.r0 + r, gv.c0 + n));
        }
    }
}

// ------------------------------------------------------------------------------------------------
// bf16 tensor-core tile product: 64 x 64 tile, 32-deep k steps, 4 warps (2 x 2, 32 x 32 each), mma.sync.m16n8k16 with fp32
// accumulators.  A arrives as fp32 and is rounded to bf16 while it is staged; W is bf16 [n][k].  Two stages: the global loads
// of step i+1 are in flight (registers) while step i multiplies.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__global__ void __launch_bounds__(128) k_gemm_bf16(const GemmArgs a) {
    pdl_enter();
    const GroupView gv = group_view(a, blockIdx.z);
    const uint32_t m0 = blockIdx.y * 64u, n0 = blockIdx.x * 64u;
    if (m0 >= gv.rows) return;
    constexpr uint32_t LD = 40;                                  // 32 + 8 bf16: fragment loads hit 32 different banks
    __shared__ __align__(16) __nv_bfloat16 As[64 * LD], Bs[64 * LD];
    __shared__ uint32_t arow[64];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u, g = lane >> 2, t = lane & 3u;
    const uint32_t wm = (warp >> 1) * 32u, wn = (warp & 1u) * 32u;
    if (tid < 64) {
        const uint32_t r = m0 + tid;
        arow[tid] = r < gv.rows ? (a.a_rows ? a.a_rows[gv.r0 + r] : gv.r0 + r) : 0xffffffffu;
    }
    __syncthreads();
    const __nv_bfloat16 *W = static_cast<const __nv_bfloat16 *>(a.W) + gv.w0;
    // staging: thread -> row tid/2, 16 consecutive k starting at (tid%2)*16, for A and for W
    const uint32_t lr = tid >> 1, lk = (tid & 1u) * 16u;
    const uint32_t ar = arow[lr];
    const float *asrc = a.A + (size_t)(ar == 0xffffffffu ? 0 : ar) * a.lda + gv.a0;
    const uint32_t wn_row = n0 + lr;
    const __nv_bfloat16 *wsrc = W + (size_t)(wn_row < a.N ? wn_row : 0) * a.ldw;
    const bool a_vec = ((reinterpret_cast<uintptr_t>(asrc) & 15u) == 0) && (a.lda % 4u == 0);
    const bool w_vec = ((reinterpret_cast<uintptr_t>(wsrc) & 15u) == 0) && (a.ldw % 8u == 0);
    float ra[16]; __align__(16) __nv_bfloat16 rw[16];
    auto fetch = [&](uint32_t k0) {
        const uint32_t kb = k0 + lk;
        if (ar != 0xffffffffu && a_vec && kb + 16u <= a.K) {
#pragma unroll
            for (uint32_t j = 0; j < 4; j++) { const float4 v = *reinterpret_cast<const float4 *>(asrc + kb + 4 * j); ra[4 * j] = v.x; ra[4 * j + 1] = v.y; ra[4 * j + 2] = v.z; ra[4 * j + 3] = v.w; }
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 16; j++) ra[j] = (ar != 0xffffffffu && kb + j < a.K) ? asrc[kb + j] : 0.0f;
        }
        if (wn_row < a.N && w_vec && kb + 16u <= a.K) {
            *reinterpret_cast<uint4 *>(rw) = *reinterpret_cast<const uint4 *>(wsrc + kb);
            *reinterpret_cast<uint4 *>(rw + 8) = *reinterpret_cast<const uint4 *>(wsrc + kb + 8);
        } else {
#pragma unroll
            for (uint32_t j = 0; j < 16; j++) rw[j] = (wn_row < a.N && kb + j < a.K) ? wsrc[kb + j] : __float2bfloat16(0.0f);
        }
    };
    auto stage = [&]() {
        __nv_bfloat16 *da = As + lr * LD + lk, *db = Bs + lr * LD + lk;
#pragma unroll
        for (uint32_t j = 0; j < 16; j += 2) {
            *reinterpret_cast<__nv_bfloat162 *>(da + j) = __floats2bfloat162_rn(ra[j], ra[j + 1]);
            *reinterpret_cast<__nv_bfloat162 *>(db + j) = __halves2bfloat162(rw[j], rw[j + 1]);
        }
    };
    float acc[2][4][4] = {};
    fetch(0);
    for (uint32_t k0 = 0; k0 < a.K; k0 += 32u) {
        stage();
        __syncthreads();
        if (k0 + 32u < a.K) fetch(k0 + 32u);
#pragma unroll
        for (uint32_t kk = 0; kk < 32; kk += 16) {
            uint32_t af[2][4], bf[4][2];
#pragma unroll
            for (uint32_t i = 0; i < 2; i++) {
                const __nv_bfloat16 *p = As + (wm + i * 16 + g) * LD + kk + 2 * t;
                af[i][0] = *reinterpret_cast<const uint32_t *>(p);
                af[i][1] = *reinterpret_cast<const uint32_t *>(p + 8 * LD);
                af[i][2] = *reinterpret_cast<const uint32_t *>(p + 8);
                af[i][3] = *reinterpret_cast<const uint32_t *>(p + 8 * LD + 8);
            }
#pragma unroll
            for (uint32_t j = 0; j < 4; j++) {
                const __nv_bfloat16 *p = Bs + (wn + j * 8 + g) * LD + kk + 2 * t;
                bf[j][0] = *reinterpret_cast<const uint32_t *>(p);
                bf[j][1] = *reinterpret_cast<const uint32_t *>(p + 8);
            }
#pragma unroll
            for (uint32_t i = 0; i < 2; i++)
#pragma unroll
                for (uint32_t j = 0; j < 4; j++) mma_bf16(acc[i][j], af[i], bf[j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (uint32_t i = 0; i < 2; i++)
#pragma unroll
        for (uint32_t j = 0; j < 4; j++)
#pragma unroll
            for (uint32_t q = 0; q < 4; q++) {
                const uint32_t r = m0 + wm + i * 16 + g + (q >> 1) * 8, n = n0 + wn + j * 8 + 2 * t + (q & 1u);
                if (r < gv.rows && n < a.N) store_c(a, a.C + (size_t)(gv.r0 + r) * a.ldc + gv.c0 + n, gated(a, epilogue(acc[i][j][q], a, gv.bias, n), gv.r0 + r, gv.c0 + n));
            }
}

// ------------------------------------------------------------------------------------------------
// matrix-vector product for up to kGemvMaxM rows per group: one warp per output column, lanes stride over k with 16-byte weight
// loads; the weight vector is read once and used for every row.  grid = (column blocks, groups).
// ------------------------------------------------------------------------------------------------
template <typename WT> struct WVec;
template <> struct WVec<float> {
    static constexpr uint32_t N = 4;
    static __device__ __forceinline__ void load(const float *p, float (&w)[N]) { const float4 v = __ldg(reinterpret_cast<const float4 *>(p)); w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w; }
};
template <> struct WVec<__nv_bfloat16> {
    static constexpr uint32_t N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&w)[N]) {
        const uint4 v = __ldg(reinterpret_cast<const uint4 *>(p));
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { w[2 * i] = __uint_as_float(u[i] << 16); w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
    }
};
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float block_sum(float v, float *red);

__device__ __forceinline__ float pick_row(const float (&v)[kGemvMaxM], int32_t i) {
    float x = v[0];
#pragma unroll
    for (int32_t j = 1; j < (int32_t)kGemvMaxM; j++) if (i == j) x = v[j];
    return x;
}
// EPI_GELU_CONV for one channel c of C: v[t] is the channel's input at row t; outputs for the rows in order, then the tail moves on
__device__ __forceinline__ void conv_rows(const GemmArgs &a, uint32_t c, uint32_t C, const float (&v)[kGemvMaxM], uint32_t rows, uint32_t r0) {
    const uint32_t K = a.cv_K;
    for (uint32_t t = 0; t < rows; t++) {
        float s = a.cv_bias[c];
        for (uint32_t j = 0; j < K; j++) {
            const int32_t src = (int32_t)t - (int32_t)(K - 1u - j);
            const float x = src >= 0 ? pick_row(v, src) : a.cv_state[(size_t)((int32_t)(K - 1u) + src) * C + c];
            s = fmaf(a.cv_taps[(size_t)c * K + j], x, s);
        }
        a.cv_out[(size_t)(r0 + t) * C + c] = s;
    }
    for (uint32_t j = 0; j + 1u < K; j++) {
        const int32_t src = (int32_t)rows - (int32_t)(K - 1u) + (int32_t)j;
        a.cv_state[(size_t)j * C + c] = src >= 0 ? pick_row(v, src) : a.cv_state[(size_t)(j + rows) * C + c];
    }
}

// EPI_CONV_RANGES for channel c of range r: taps [C][K], bias optional, tail [K - 1][C], out [rows][C], silu when r.act
__device__ __forceinline__ void conv_range_rows(const GemmArgs::ConvRange &r, uint32_t c, const float (&v)[kGemvMaxM], uint32_t rows, uint32_t r0) {
    const uint32_t K = r.K, C = r.n1 - r.n0;
    for (uint32_t t = 0; t < rows; t++) {
        float s = r.bias ? r.bias[c] : 0.0f;
        for (uint32_t j = 0; j < K; j++) {
            const int32_t src = (int32_t)t - (int32_t)(K - 1u - j);
            const float x = src >= 0 ? pick_row(v, src) : r.state[(size_t)((int32_t)(K - 1u) + src) * C + c];
            s = fmaf(r.taps[(size_t)c * K + j], x, s);
        }
        if (r.act) s = s / (1.0f + expf(-s));
        r.out[(size_t)(r0 + t) * C + c] = s;
    }
    for (uint32_t j = 0; j + 1u < K; j++) {
        const int32_t src = (int32_t)rows - (int32_t)(K - 1u) + (int32_t)j;
        r.state[(size_t)j * C + c] = src >= 0 ? pick_row(v, src) : r.state[(size_t)(j + rows) * C + c];
    }
}

// dot products of one weight row with up to kGemvMaxM activation rows, summed over the warp's lanes: every lane returns the totals.
// sc[i] / nw: the optional RMS-norm prologue (A[i][k] * sc[i] * nw[k]); pc: the optional PolyNorm prologue, pc[i] = (a / rms(z), b / rms(z^2),
// c / rms(z^3), e) of row i; rnd: round the activation to bf16 first.
struct PolyRow { float r1, r2, r3, e; };
__device__ __forceinline__ float poly_of(float x, const PolyRow &p) { return fmaf(p.r1, x, fmaf(p.r2, x * x, fmaf(p.r3, x * x * x, p.e))); }
// GN: the scale of row i at column k is gsc[i * 32 + k / plen] (a norm in equal parts) instead of sc[i]
template <typename WT, bool POLY = false, bool GN = false>
__device__ __forceinline__ void warp_dots(const WT *wr, const float *(&ap)[kGemvMaxM], uint32_t rows, uint32_t K, uint32_t kvec, const float (&sc)[kGemvMaxM],
                                          const float *nw, bool rnd, uint32_t lane, float (&acc)[kGemvMaxM], const PolyRow *pc = nullptr,
                                          const float *gsc = nullptr, uint32_t plen = 1) {
    constexpr uint32_t VN = WVec<WT>::N;
#pragma unroll
    for (uint32_t i = 0; i < kGemvMaxM; i++) acc[i] = 0.0f;
#pragma unroll 4
    for (uint32_t k = lane * VN; k < kvec; k += 32u * VN) {
        float w[VN];
        WVec<WT>::load(wr + k, w);
#pragma unroll
        for (uint32_t i = 0; i < kGemvMaxM; i++) {
            if (i < rows) {
#pragma unroll
                for (uint32_t j = 0; j < VN; j += 4) {
                    float4 x = *reinterpret_cast<const float4 *>(ap[i] + k + j);
                    if (nw) {
                        const float si = GN ? gsc[i * 32u + (k + j) / plen] : sc[i];
                        const float4 g = __ldg(reinterpret_cast<const float4 *>(nw + k + j)); x.x = x.x * si * g.x; x.y = x.y * si * g.y; x.z = x.z * si * g.z; x.w = x.w * si * g.w;
                    }
                    if (POLY && pc) { x.x = poly_of(x.x, pc[i]); x.y = poly_of(x.y, pc[i]); x.z = poly_of(x.z, pc[i]); x.w = poly_of(x.w, pc[i]); }
                    if (rnd) { x.x = round_bf16(x.x); x.y = round_bf16(x.y); x.z = round_bf16(x.z); x.w = round_bf16(x.w); }
                    acc[i] = fmaf(w[j], x.x, acc[i]); acc[i] = fmaf(w[j + 1], x.y, acc[i]);
                    acc[i] = fmaf(w[j + 2], x.z, acc[i]); acc[i] = fmaf(w[j + 3], x.w, acc[i]);
                }
            }
        }
    }
    for (uint32_t k = kvec + lane; k < K; k += 32u) {
        const float w = wval(wr + k);
#pragma unroll
        for (uint32_t i = 0; i < kGemvMaxM; i++)
            if (i < rows) {
                float x = ap[i][k];
                if (nw) x = x * (GN ? gsc[i * 32u + k / plen] : sc[i]) * nw[k];
                if (POLY && pc) x = poly_of(x, pc[i]);
                acc[i] = fmaf(w, rnd ? round_bf16(x) : x, acc[i]);
            }
    }
#pragma unroll
    for (uint32_t i = 0; i < kGemvMaxM; i++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
}

// EXT 1: the instance that also knows the convolution-range epilogue, EXT 2: the PolyNorm prologue, EXT 3: the gated pair, EXT 4: the
// norm in equal parts, EXT 5: the plain product with the residual epilogue, which EXT 4 knows too (registers the plain one keeps)
template <typename WT, int EXT = 0>
__device__ __forceinline__ void gemv_body(const GemmArgs &a, float *red) {
    const GroupView gv = group_view(a, blockIdx.y);
    if (gv.rows == 0) return;
    const uint32_t rows = gv.rows < kGemvMaxM ? gv.rows : kGemvMaxM;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), nwarps = gridDim.x * (blockDim.x >> 5);
    const WT *W = static_cast<const WT *>(a.W) + gv.w0;
    const float *ap[kGemvMaxM];
    float sc[kGemvMaxM];
    bool vec = (a.ldw % WVec<WT>::N == 0) && ((reinterpret_cast<uintptr_t>(W) & 15u) == 0);
#pragma unroll
    for (uint32_t i = 0; i < kGemvMaxM; i++) {
        const uint32_t r = gv.r0 + (i < rows ? i : 0);
        ap[i] = a.A + (size_t)(a.a_rows ? a.a_rows[r] : r) * a.lda + gv.a0;
        vec = vec && ((reinterpret_cast<uintptr_t>(ap[i]) & 15u) == 0);
        sc[i] = 1.0f;
    }
    __shared__ float gsc[EXT == 4 ? kGemvMaxM * 32 : 1];
    const uint32_t plen = EXT == 4 ? a.K / a.a_parts : 1u;
    if (EXT == 4) {          // a warp per (row, part): the part's root mean square
        for (uint32_t job = threadIdx.x >> 5; job < rows * a.a_parts; job += blockDim.x >> 5) {
            const uint32_t i = job / a.a_parts, p = job % a.a_parts;
            const float *src = a.A + (size_t)(a.a_rows ? a.a_rows[gv.r0 + i] : gv.r0 + i) * a.lda + gv.a0 + p * plen;
            float s = 0.0f;
            for (uint32_t k = lane * 4u; k < plen; k += 128u) { const float4 q = *reinterpret_cast<const float4 *>(src + k); s = fmaf(q.x, q.x, fmaf(q.y, q.y, fmaf(q.z, q.z, fmaf(q.w, q.w, s)))); }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) gsc[i * 32u + p] = 1.0f / sqrtf(s / (float)plen + a.a_eps);
        }
        __syncthreads();
    } else if (a.a_norm_w) {          // rows is the same for every thread of the block
#pragma unroll
        for (uint32_t i = 0; i < kGemvMaxM; i++)
            if (i < rows) {
                float s = 0.0f;
                for (uint32_t k = threadIdx.x; k < a.K; k += blockDim.x) s = fmaf(ap[i][k], ap[i][k], s);
                s = block_sum(s, red);
                sc[i] = 1.0f / sqrtf(s / (float)a.K + a.a_eps);
            }
    }
    PolyRow pc[EXT == 2 ? kGemvMaxM : 1];
    if (EXT == 2 && a.a_poly) {
#pragma unroll
        for (uint32_t i = 0; i < kGemvMaxM; i++)
            if (i < rows) {
                float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
                const uint32_t k4 = vec ? a.K & ~3u : 0u;          // 16-byte loads where the row allows them
#pragma unroll 4
                for (uint32_t k = threadIdx.x * 4u; k < k4; k += blockDim.x * 4u) {
                    const float4 q = *reinterpret_cast<const float4 *>(ap[i] + k);
                    const float w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) { const float v2 = w[j] * w[j], v3 = v2 * w[j]; s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6); }
                }
                for (uint32_t k = k4 + threadIdx.x; k < a.K; k += blockDim.x) { const float v = ap[i][k], v2 = v * v, v3 = v2 * v; s2 += v2; s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6); }
                s2 = block_sum(s2, red); s4 = block_sum(s4, red); s6 = block_sum(s6, red);
                pc[i].r1 = a.a_poly[0] / sqrtf(s2 / (float)a.K + a.a_eps); pc[i].r2 = a.a_poly[1] / sqrtf(s4 / (float)a.K + a.a_eps);
                pc[i].r3 = a.a_poly[2] / sqrtf(s6 / (float)a.K + a.a_eps); pc[i].e = a.a_poly[3];
            }
    }
    const uint32_t kvec = vec ? (a.K / WVec<WT>::N) * WVec<WT>::N : 0u;
    for (uint32_t n = warp0; n < a.N; n += nwarps) {
        float acc[kGemvMaxM];
        warp_dots<WT, EXT == 2, EXT == 4>(W + (size_t)n * a.ldw, ap, rows, a.K, kvec, sc, a.a_norm_w, a.round_a != 0, lane, acc, (EXT == 2 && a.a_poly) ? pc : nullptr, gsc, plen);
        if (EXT == 3) {          // the up row of the pair, then act(s g) (s u)
            float up[kGemvMaxM];
            warp_dots<WT, false>(W + (size_t)(a.N + n) * a.ldw, ap, rows, a.K, kvec, sc, nullptr, a.round_a != 0, lane, up);
            if (lane != 0) continue;
#pragma unroll
            for (uint32_t i = 0; i < kGemvMaxM; i++)
                if (i < rows) {
                    const float s = a.row_scale ? a.row_scale[gv.r0 + i] : 1.0f, g = acc[i] * s, u = up[i] * s;
                    store_c(a, a.C + (size_t)(gv.r0 + i) * a.ldc + gv.c0 + n, a.glu == 3u ? clamped_glu(g, u, a.glu_limit) : (a.glu == 2u ? g / (1.0f + expf(-g)) : gelu_tanh(g)) * u);
                }
            continue;
        }
        if (lane != 0) continue;
        if (EXT == 1 && a.epi == EPI_CONV_RANGES) {
            bool done = false;
#pragma unroll
            for (int ri = 0; ri < 2; ri++)
                if (n >= a.cr[ri].n0 && n < a.cr[ri].n1) { conv_range_rows(a.cr[ri], n - a.cr[ri].n0, acc, rows, gv.r0); done = true; }
            if (done) continue;
        }
        if (a.epi == EPI_GELU_CONV && n >= a.split) {
            float v[kGemvMaxM];
#pragma unroll
            for (uint32_t i = 0; i < kGemvMaxM; i++) v[i] = acc[i] + (gv.bias ? gv.bias[n] : 0.0f);
            conv_rows(a, n - a.split, a.N - a.split, v, rows, gv.r0);
            continue;
        }
#pragma unroll
        for (uint32_t i = 0; i < kGemvMaxM; i++)
            if (i < rows) {
                const float v = epilogue(acc[i], a, gv.bias, n);
                if ((EXT == 4 || EXT == 5) && a.res_x) {
                    const size_t at = (size_t)(gv.r0 + i) * a.N + n;
                    const float xv = a.res_x[at] + fmaf(tanhf(a.res_pa * v), a.res_pw[n], a.res_pb[n]);
                    a.res_x[at] = xv;
                    if (a.res_keep) a.res_keep[at] = xv;
                    if (a.res_out) a.res_out[at] = fmaf(tanhf(a.res_na * xv), a.res_nw[n], a.res_nb[n]);
                } else store_c(a, a.C + (size_t)(gv.r0 + i) * a.ldc + gv.c0 + n, gated(a, v, gv.r0 + i, gv.c0 + n));
            }
    }
}

// the weight rows this block's warps will read first (plain and fixed-group products; a routed product learns its groups from the
// kernel before and asks for nothing)
template <typename WT>
__device__ __forceinline__ void gemv_prefetch(const GemmArgs &a) {
    if (a.g_off) return;
    const WT *W = static_cast<const WT *>(a.W) + (uint64_t)blockIdx.y * a.w_gstride;
    prefetch_weight_rows(W, sizeof(WT), a.ldw, a.K, a.N, blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), gridDim.x * (blockDim.x >> 5), 2u);
}
template <typename WT>
__global__ void __launch_bounds__(256) k_gemv(const GemmArgs a) {
    pdl_launch_next();
    gemv_prefetch<WT>(a);
    pdl_wait();
    __shared__ float red[32];
    gemv_body<WT>(a, red);
}
template <typename WT, int EXT>
__global__ void __launch_bounds__(256) k_gemv_ext(const GemmArgs a) {
    pdl_launch_next();
    gemv_prefetch<WT>(a);
    pdl_wait();
    __shared__ float red[32];
    gemv_body<WT, EXT>(a, red);
}

// ------------------------------------------------------------------------------------------------
// block-wide sum (blockDim.x a multiple of 32, <= 1024); every thread gets the result
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float block_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.0f;
    for (uint32_t w = 0; w < (blockDim.x >> 5); w++) s += red[w];
    return s;
}

// x[t] = embed[tokens[base + t]]; x0 keeps a copy when a later pass adds the embedding output again.  base = *pos_ptr when given: a
// captured decode step reads "the token at the sequence's present position" without a host-side argument
template <typename WT>
__global__ void k_embed(const uint32_t *__restrict__ tokens, const uint32_t *__restrict__ pos_ptr, const WT *__restrict__ embed, float *__restrict__ x,
                        float *__restrict__ x0, uint32_t E) {
    pdl_enter();
    const uint32_t t = blockIdx.x;
    const WT *src = embed + (size_t)tokens[t + (pos_ptr ? *pos_ptr : 0u)] * E;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) {
        const float v = wval(src + i);
        x[(size_t)t * E + i] = v;
        if (x0) x0[(size_t)t * E + i] = v;
    }
}

__global__ void k_add(float *__restrict__ x, const float *__restrict__ y, size_t n) {
    pdl_enter();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] += y[i];
}

// Scalar-gain RMS norm of x with two gains at once (mixer input, feed-forward input) and the token shift of the mixer input:
//   n1[t] = x[t] / rms(x[t]) * g1,  hm[t] = n1[t] + (n1[t-1] - n1[t]) * mu,  n1[-1] = the state (zeros at the start of a sequence),
//   h2[t] = x[t] / rms(x[t]) * g2.   The state becomes n1[T-1].
// Block b handles token b; block 0 also handles the LAST token after token 0, so the one reader and the one writer of the state
// are the same block, in that order.
struct NormShiftArgs {
    const float *x; const float *g1, *g2, *mu; float *state; float *hm, *h2;
    uint32_t T, E; float eps;
};
__device__ __forceinline__ void norm_shift_token(const NormShiftArgs &a, uint32_t t, float *red) {
    const float *xt = a.x + (size_t)t * a.E, *xp = t ? xt - a.E : nullptr;
    float s = 0.0f, sp = 0.0f;
    for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) { const float v = xt[i]; s = fmaf(v, v, s); if (xp) { const float u = xp[i]; sp = fmaf(u, u, sp); } }
    s = block_sum(s, red);
    sp = block_sum(sp, red);
    const float rinv = 1.0f / sqrtf(s / (float)a.E + a.eps), rinvp = 1.0f / sqrtf(sp / (float)a.E + a.eps);
    const float g1 = *a.g1, g2 = a.g2 ? *a.g2 : 0.0f;
    for (uint32_t i = threadIdx.x; i < a.E; i += blockDim.x) {
        const float u = xt[i] * rinv;
        const float n1 = u * g1;
        const float prev = xp ? xp[i] * rinvp * g1 : a.state[i];
        a.hm[(size_t)t * a.E + i] = a.mu ? n1 + (prev - n1) * a.mu[i] : n1;
        if (a.h2) a.h2[(size_t)t * a.E + i] = u * g2;
        if (t + 1 == a.T) a.state[i] = n1;
    }
}
__global__ void __launch_bounds__(256) k_norm_shift(const NormShiftArgs a) {
    pdl_enter();
    __shared__ float red[32];
    norm_shift_token(a, blockIdx.x, red);
    if (blockIdx.x == 0 && a.T > 1) { __syncthreads(); norm_shift_token(a, a.T - 1, red); }
}

// causal per-channel convolution: u[t,c] = b[c] + sum_j taps[c,j] * v[t - (K-1-j), c]; inputs before this portion come from the
// state (the last K-1 inputs of the sequence so far, oldest first; zeros at the start)
// bias may be null; ldu: row stride of u (0: C); act 1: silu on the output
struct ConvArgs { const float *v; uint32_t ldv; const float *taps, *bias; float *state; float *u; uint32_t T, C, K; uint32_t ldu, act; };
__global__ void k_conv(const ConvArgs a) {
    pdl_enter();
    const size_t total = (size_t)a.T * a.C;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / a.C), c = (uint32_t)(i % a.C);
        float s = a.bias ? a.bias[c] : 0.0f;
        for (uint32_t j = 0; j < a.K; j++) {
            const int64_t src = (int64_t)t - (int64_t)(a.K - 1 - j);
            const float v = src >= 0 ? a.v[(size_t)src * a.ldv + c] : a.state[(size_t)((int64_t)(a.K - 1) + src) * a.C + c];
            s = fmaf(a.taps[(size_t)c * a.K + j], v, s);
        }
        if (a.act) s = s / (1.0f + expf(-s));
        a.u[(size_t)t * (a.ldu ? a.ldu : a.C) + c] = s;
    }
}
// after k_conv: the tail becomes the last K-1 inputs, this portion included
__global__ void k_conv_state(const ConvArgs a) {
    pdl_enter();
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    for (uint32_t j = 0; j + 1 < a.K; j++) {
        const int64_t src = (int64_t)a.T - (int64_t)(a.K - 1) + j;
        a.state[(size_t)j * a.C + c] = src >= 0 ? a.v[(size_t)src * a.ldv + c] : a.state[(size_t)(j + a.T) * a.C + c];
    }
}

// real-gated linear recurrent unit, one thread per channel, tokens in order:
//   a = exp(-c_decay * r * softplus(lam)),  S <- a S + sqrt(1 - a^2) * (i * u),  out = S * y
struct ScanArgs { const float *gates; uint32_t ldg; const float *u; const float *y; uint32_t ldy; const float *lam; float *S; float *out; uint32_t T, C; float c_decay; };
__global__ void k_rglru_scan(const ScanArgs a) {
    pdl_enter();
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.C) return;
    const float sp = softplusf_(a.lam[c]);
    float S = a.S[c];
    for (uint32_t t = 0; t < a.T; t++) {
        const float r = a.gates[(size_t)t * a.ldg + c], i = a.gates[(size_t)t * a.ldg + a.C + c];
        const float la = -a.c_decay * r * sp;
        const float av = expf(la);
        S = av * S + sqrtf(1.0f - av * av) * (i * a.u[(size_t)t * a.C + c]);
        a.out[(size_t)t * a.C + c] = S * a.y[(size_t)t * a.ldy + c];
    }
    a.S[c] = S;
}

// The same recurrence for long portions, parallel over time: the portion is cut into blockDim.y segments.  A thread (channel,
// segment) first composes its segment's affine map S -> P S + Q, the segment-0 threads chain the maps to every segment's entry
// state (and the portion's final state), then each thread replays its segment from its entry state and writes the outputs.
__global__ void __launch_bounds__(1024) k_rglru_scan_par(const ScanArgs a) {
    pdl_enter();
    __shared__ float P[32][33], Q[32][33];
    const uint32_t x = threadIdx.x, seg = threadIdx.y, nseg = blockDim.y, c = blockIdx.x * 32u + x;
    const uint32_t Ls = (a.T + nseg - 1u) / nseg, t0 = min(a.T, seg * Ls), t1 = min(a.T, t0 + Ls);
    const bool live = c < a.C;
    const float sp = live ? softplusf_(a.lam[c]) : 0.0f;
    float p = 1.0f, q = 0.0f;
    if (live)
        for (uint32_t t = t0; t < t1; t++) {
            const float r = a.gates[(size_t)t * a.ldg + c], i = a.gates[(size_t)t * a.ldg + a.C + c];
            const float av = expf(-a.c_decay * r * sp);
            q = av * q + sqrtf(1.0f - av * av) * (i * a.u[(size_t)t * a.C + c]);
            p *= av;
        }
    P[seg][x] = p; Q[seg][x] = q;
    __syncthreads();
    if (seg == 0 && live) {
        float s = a.S[c];
        for (uint32_t g = 0; g < nseg; g++) { const float pg = P[g][x], qg = Q[g][x]; P[g][x] = s; s = pg * s + qg; }
        a.S[c] = s;
    }
    __syncthreads();
    if (!live) return;
    float S = P[seg][x];
    for (uint32_t t = t0; t < t1; t++) {
        const float r = a.gates[(size_t)t * a.ldg + c], i = a.gates[(size_t)t * a.ldg + a.C + c];
        const float av = expf(-a.c_decay * r * sp);
        S = av * S + sqrtf(1.0f - av * av) * (i * a.u[(size_t)t * a.C + c]);
        a.out[(size_t)t * a.C + c] = S * a.y[(size_t)t * a.ldy + c];
    }
}

// Gates and recurrence of a short portion (<= kGemvMaxM tokens) in one launch: a warp per channel c of block b computes both gate
// rows of its channel, r = sigmoid(ra[b][c] . u_b + bias) and i = sigmoid(ri[b][c] . u_b + bias), for every token, then runs the
// recurrence of k_rglru_scan for that channel.  W = [ra blocks | ri blocks], each block [bs][bs]; bias likewise.
struct GatesScanArgs { const float *u; const void *W; const float *bias; const float *y; uint32_t ldy; const float *lam; float *S; float *out; uint32_t T, C, bs; float c_decay; uint32_t round_a; };
template <typename WT>
__global__ void __launch_bounds__(256) k_rglru_gates_scan(const GatesScanArgs a) {
    pdl_launch_next();
    {   // both gate rows of this warp's channel
        const uint32_t c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        if (c < a.C) {
            prefetch_weight_rows(a.W, sizeof(WT), a.bs, a.bs, a.C, c, a.C, 1u);
            prefetch_weight_rows(static_cast<const WT *>(a.W) + (size_t)a.C * a.bs, sizeof(WT), a.bs, a.bs, a.C, c, a.C, 1u);
        }
    }
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31u, c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (c >= a.C) return;
    const uint32_t b = c / a.bs, rows = a.T < kGemvMaxM ? a.T : kGemvMaxM;
    const WT *W = static_cast<const WT *>(a.W);
    const WT *wr = W + (size_t)c * a.bs, *wi = W + (size_t)(a.C + c) * a.bs;
    const float *ap[kGemvMaxM];
    float sc[kGemvMaxM];
    bool vec = (a.bs % WVec<WT>::N == 0) && ((reinterpret_cast<uintptr_t>(W) & 15u) == 0);
#pragma unroll
    for (uint32_t i = 0; i < kGemvMaxM; i++) {
        ap[i] = a.u + (size_t)(i < rows ? i : 0) * a.C + (size_t)b * a.bs;
        vec = vec && ((reinterpret_cast<uintptr_t>(ap[i]) & 15u) == 0);
        sc[i] = 1.0f;
    }
    const uint32_t kvec = vec ? (a.bs / WVec<WT>::N) * WVec<WT>::N : 0u;
    float gr[kGemvMaxM], gi[kGemvMaxM];
    warp_dots<WT>(wr, ap, rows, a.bs, kvec, sc, nullptr, a.round_a != 0, lane, gr);
    warp_dots<WT>(wi, ap, rows, a.bs, kvec, sc, nullptr, a.round_a != 0, lane, gi);
    if (lane != 0) return;
    const float sp = softplusf_(a.lam[c]), br = a.bias[c], bi = a.bias[a.C + c];
    float S = a.S[c];
#pragma unroll
    for (uint32_t t = 0; t < kGemvMaxM; t++) {
        if (t < rows) {
            const float r = sigmoidf_(gr[t] + br), i = sigmoidf_(gi[t] + bi);
            const float av = expf(-a.c_decay * r * sp);
            S = av * S + sqrtf(1.0f - av * av) * (i * a.u[(size_t)t * a.C + c]);
            a.out[(size_t)t * a.C + c] = S * a.y[(size_t)t * a.ldy + c];
        }
    }
    a.S[c] = S;
}

// vector-gain RMS norms of the two latents of one token: z = [query latent | key/value latent]; the query latent goes to cq, the
// key/value latent into the sequence's cache page of position pos0 + t
struct LatentNormArgs { const float *z; uint32_t ldz; const float *wq, *wkv; float *cq; float *cache; const uint32_t *table; uint32_t QR, R, pos0; float eps; const uint32_t *pos_ptr; };
// the key/value latent of token t: normed, into the cache page of its position
__device__ __forceinline__ void latent_kv_row(const LatentNormArgs &a, uint32_t t, float *red) {
    const float *z = a.z + (size_t)t * a.ldz + a.QR;
    float s2 = 0.0f;
    for (uint32_t i = threadIdx.x; i < a.R; i += blockDim.x) s2 = fmaf(z[i], z[i], s2);
    s2 = block_sum(s2, red);
    const float rk = 1.0f / sqrtf(s2 / (float)a.R + a.eps);
    const uint32_t pos = a.pos0 + t + (a.pos_ptr ? *a.pos_ptr : 0u);
    float *row = a.cache + ((size_t)a.table[pos / kPage] * kPage + pos % kPage) * a.R;
    for (uint32_t i = threadIdx.x; i < a.R; i += blockDim.x) row[i] = z[i] * rk * a.wkv[i];
}
__global__ void __launch_bounds__(128) k_latent_norm(const LatentNormArgs a) {
    pdl_enter();
    __shared__ float red[32];
    const uint32_t t = blockIdx.x;
    const float *z = a.z + (size_t)t * a.ldz;
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < a.QR; i += blockDim.x) s = fmaf(z[i], z[i], s);
    s = block_sum(s, red);
    const float rq = 1.0f / sqrtf(s / (float)a.QR + a.eps);
    for (uint32_t i = threadIdx.x; i < a.QR; i += blockDim.x) a.cq[(size_t)t * a.QR + i] = z[i] * rq * a.wq[i];
    latent_kv_row(a, t, red);
}
// Short portions: the query latent's norm is the prologue of the query up-projection (GemmArgs::a_norm_w) and the last block of
// that product also norms and caches the key/value latents, so the two norms cost no launch of their own.
struct GemvLatentArgs { GemmArgs g; LatentNormArgs n; uint32_t T; };
template <typename WT>
__global__ void __launch_bounds__(256) k_gemv_latent(const GemvLatentArgs a) {
    pdl_launch_next();
    gemv_prefetch<WT>(a.g);
    pdl_wait();
    __shared__ float red[32];
    if (blockIdx.x == gridDim.x - 1u && blockIdx.y == 0)
        for (uint32_t t = 0; t < a.T; t++) latent_kv_row(a.n, t, red);
    gemv_body<WT>(a.g, red);
}

// Softmax attention over cached latents.  qa[t][h][:] is head h's query already multiplied into latent space (q_h^T W_uk,h), so
// score(t, j) = scale * qa[t][h] . c_j and the head's output in latent space is sum_j p_j c_j (multiplied by W_uv,h afterwards):
// the latent row is key and value at once and a block reads it once for QT query tokens x kAttnWarps heads.  Causal: query t sees
// keys 0 .. pos + t, pos = pos0 (+ *pos_ptr in a captured decode step).
// grid = (query tiles of QT tokens, key splits, head groups); one warp per head; lanes = keys for the scores, = latent columns for
// the weighted sum; online softmax in fp32.  A key tile (one cache page) is fetched with all of a thread's 16-byte loads in flight
// at once.  With one split the normalised result is written; otherwise partial (o, m, l) triples, merged at the end.
struct AttnArgs {
    const float *qa; const float *cache; const uint32_t *table; float *out; float *part;
    uint32_t T, H, R, pos0, nsplit; float scale; const uint32_t *pos_ptr;
    uint32_t *tickets;      // nsplit > 1: one zeroed counter per (query tile, head group); the block that draws the last ticket merges
    // Options (a design without them passes 0, kAttnNoWindow, null).  KX: a cache row is [R latent columns | KX more key columns] and a
    // query row likewise; the score runs over all R + KX columns (a rotated key part shared by the heads beside the latent), the
    // weighted sum over the R latent columns only.  window: query i sees key j only while i - j < window.  sink: one number per head
    // that joins the softmax denominator as exp(sink_h), with no key and no value.
    uint32_t KX, window; const float *sink;
};
constexpr uint32_t kAttnNoWindow = 1u << 30;
// EXACT: the latent rank is RCH * 32 (64, 128, 256, 512): R is a compile-time constant, so row offsets are immediates, the
// divisions of the staging loops are shifts and the column guards vanish.
// Two blocks per SM (128 registers) where the shared memory of a prefill instance fits twice; measured faster at rank 256 with 8 queries,
// slower where the second block cannot be resident anyway (rank 512).
constexpr bool attn_two_blocks(int rch, int qt, bool exact) {
    return exact && qt > 1 && ((size_t)qt * kAttnWarps * rch * 32 + (size_t)kPage * (rch * 32 + 4)) * 4 <= 112u * 1024u;
}
// EXT: the instance that knows the options (extra key columns, window, sink); the plain one ignores them and keeps its registers
template <int RCH, int QT, bool EXACT, bool EXT = false>
__global__ void __launch_bounds__(kAttnWarps * 32, attn_two_blocks(RCH, QT, EXACT) ? 2 : 1) k_latent_attn(const AttnArgs a) {
    pdl_enter();
    const uint32_t a_KX = EXT ? a.KX : 0u, a_window = EXT ? a.window : kAttnNoWindow;
    const float *a_sink = EXT ? a.sink : nullptr;
    extern __shared__ __align__(16) float sm[];
    const uint32_t tq0 = blockIdx.x * QT, split = blockIdx.y, h0 = blockIdx.z * kAttnWarps;
    const uint32_t nq = min((uint32_t)QT, a.T - tq0);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, h = h0 + warp;
    const uint32_t R = EXACT ? (uint32_t)RCH * 32u : a.R;
    const uint32_t RS = EXT ? R + a_KX : R;       // row length of the cache and of the queries (R itself, a constant, without extra key columns)
    const bool vec = (R % 4u) == 0 && (RS % 4u) == 0;      // 16-byte shared-memory rows: (R + 4) / 4 is odd for R % 8 == 0, so 8 lanes hit 8 bank groups
    const uint32_t LDC = vec ? RS + 4u : RS + 1u;
    float *q_s = sm;                               // [QT][kAttnWarps][RS]
    float *c_s = sm + QT * kAttnWarps * RS;        // [kPage][LDC]
    const uint32_t pos = a.pos0 + (a.pos_ptr ? *a.pos_ptr : 0u);
    const uint32_t nkeys = pos + tq0 + nq, tiles = (nkeys + kPage - 1u) / kPage;      // keys of the block's last query
    // the oldest key the block's FIRST query sees: tiles before it hold nothing for any query of the block
    const uint32_t tile_first = EXT ? (pos + tq0 + 1u > a_window ? pos + tq0 + 1u - a_window : 0u) / kPage : 0u;
    const uint32_t tps = (tiles - tile_first + a.nsplit - 1u) / a.nsplit;
    const uint32_t tile_lo = tile_first + split * tps, tile_hi = min(tiles, tile_lo + tps);
    if (vec) {          // a query token's kAttnWarps heads are contiguous in qa: 16-byte copies, all of a thread's loads in flight
        const uint32_t per = kAttnWarps * RS / 4u, live = (min(a.H, h0 + kAttnWarps) - h0) * RS / 4u;
#pragma unroll 4
        for (uint32_t i = threadIdx.x; i < QT * per; i += blockDim.x) {
            const uint32_t qi = i / per, rem = i % per;
            float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (qi < nq && rem < live) v = *(reinterpret_cast<const float4 *>(a.qa + ((size_t)(tq0 + qi) * a.H + h0) * RS) + rem);
            reinterpret_cast<float4 *>(q_s)[i] = v;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < QT * kAttnWarps * RS; i += blockDim.x) {
            const uint32_t qi = i / (kAttnWarps * RS), rem = i % (kAttnWarps * RS), hh = h0 + rem / RS;
            q_s[i] = (qi < nq && hh < a.H) ? a.qa[((size_t)(tq0 + qi) * a.H + hh) * RS + rem % RS] : 0.0f;
        }
    }
    float m[QT], l[QT], o[QT][RCH];
#pragma unroll
    for (int qi = 0; qi < QT; qi++) {
        m[qi] = -INFINITY; l[qi] = 0.0f;
#pragma unroll
        for (int c = 0; c < RCH; c++) o[qi][c] = 0.0f;
    }
    for (uint32_t tile = tile_lo; tile < tile_hi; tile++) {
        __syncthreads();
        const float *src = a.cache + (size_t)a.table[tile] * kPage * RS;
        const uint32_t nk = min(kPage, nkeys - tile * kPage);
        if (vec) {
            const uint32_t n4 = nk * RS / 4u;
            const float4 *src4 = reinterpret_cast<const float4 *>(src);
            for (uint32_t base = 0; base < n4; base += 8u * kAttnWarps * 32u) {
                float4 v[8];
#pragma unroll
                for (int k = 0; k < 8; k++) { const uint32_t i = base + k * kAttnWarps * 32u + threadIdx.x; if (i < n4) v[k] = __ldg(src4 + i); }
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const uint32_t i = base + k * kAttnWarps * 32u + threadIdx.x;
                    if (i < n4) *reinterpret_cast<float4 *>(c_s + (i * 4u / RS) * LDC + (i * 4u) % RS) = v[k];
                }
            }
        } else {
            for (uint32_t i = threadIdx.x; i < nk * RS; i += blockDim.x) c_s[(i / RS) * LDC + i % RS] = src[i];
        }
        __syncthreads();
        if (h >= a.H) continue;
        uint32_t nkq[QT], lokq[QT];     // keys [lokq, nkq) of this tile are the ones each query sees (nkq 0: the tile lies after the query)
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            const uint32_t kq = pos + tq0 + qi + 1u;
            nkq[qi] = ((uint32_t)qi < nq && kq > tile * kPage) ? min(nk, kq - tile * kPage) : 0u;
            const uint32_t oldest = kq > a_window ? kq - a_window : 0u;
            lokq[qi] = (EXT && oldest > tile * kPage) ? oldest - tile * kPage : 0u;
        }
        float sc[QT];
#pragma unroll
        for (int qi = 0; qi < QT; qi++) sc[qi] = 0.0f;
        const float *cr = c_s + lane * LDC;         // lanes past nk read rows of an earlier tile: their scores are masked below
        if (vec) {
            float sc4[4] = {0.0f, 0.0f, 0.0f, 0.0f};      // a single query: four independent partial sums instead of one long chain
            const float4 *c4 = reinterpret_cast<const float4 *>(cr);
            auto score4 = [&](uint32_t r4) {
                const float4 cv = c4[r4];
#pragma unroll
                for (int qi = 0; qi < QT; qi++) {
                    const float4 qv = reinterpret_cast<const float4 *>(q_s + ((size_t)qi * kAttnWarps + warp) * RS)[r4];
                    if (QT == 1) { sc4[0] = fmaf(qv.x, cv.x, sc4[0]); sc4[1] = fmaf(qv.y, cv.y, sc4[1]); sc4[2] = fmaf(qv.z, cv.z, sc4[2]); sc4[3] = fmaf(qv.w, cv.w, sc4[3]); }
                    else sc[qi] = fmaf(qv.w, cv.w, fmaf(qv.z, cv.z, fmaf(qv.y, cv.y, fmaf(qv.x, cv.x, sc[qi]))));
                }
            };
            for (uint32_t r4 = 0; r4 < R / 4u; r4++) score4(r4);
            if (EXT) for (uint32_t r4 = R / 4u; r4 < RS / 4u; r4++) score4(r4);      // the extra key columns
            if (QT == 1) sc[0] = (sc4[0] + sc4[1]) + (sc4[2] + sc4[3]);
        } else {
            for (uint32_t r = 0; r < RS; r++) {
                const float cv = cr[r];
#pragma unroll
                for (int qi = 0; qi < QT; qi++) sc[qi] = fmaf(q_s[((size_t)qi * kAttnWarps + warp) * RS + r], cv, sc[qi]);
            }
        }
        float p[QT];
        uint32_t nkmax = 0;
#pragma unroll
        for (int qi = 0; qi < QT; qi++) {
            const bool seen = lane < nkq[qi] && lane >= lokq[qi];
            const float s = seen ? sc[qi] * a.scale : -INFINITY;
            float tm = s;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, off));
            const float mn = fmaxf(m[qi], tm);
            const float corr = mn == -INFINITY ? 1.0f : expf(m[qi] - mn);
            p[qi] = seen ? expf(s - mn) : 0.0f;
            float ps = p[qi];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            l[qi] = l[qi] * corr + ps;
            m[qi] = mn;
#pragma unroll
            for (int c = 0; c < RCH; c++) o[qi][c] *= corr;
            nkmax = max(nkmax, nkq[qi]);
        }
        for (uint32_t j = 0; j < nkmax; j++) {
            float pj[QT];
#pragma unroll
            for (int qi = 0; qi < QT; qi++) pj[qi] = __shfl_sync(0xffffffffu, p[qi], j);
            const float *cj = c_s + j * LDC;
#pragma unroll
            for (int c = 0; c < RCH; c++) {
                const uint32_t r = lane + 32u * c;
                if (r < R) {
                    const float cv = cj[r];
#pragma unroll
                    for (int qi = 0; qi < QT; qi++) o[qi][c] = fmaf(pj[qi], cv, o[qi][c]);
                }
            }
        }
    }
#pragma unroll
    for (int qi = 0; qi < QT; qi++) {
        if ((uint32_t)qi >= nq || h >= a.H) continue;
        const uint32_t t = tq0 + qi;
        if (a.nsplit == 1) {
            float den = l[qi], ow = 1.0f;
            if (a_sink) {      // the sink joins the denominator, under the common maximum
                const float sk = a_sink[h], mm = fmaxf(m[qi], sk);
                ow = expf(m[qi] - mm); den = l[qi] * ow + expf(sk - mm);
            }
            const float inv = ow / den;
#pragma unroll
            for (int c = 0; c < RCH; c++) { const uint32_t r = lane + 32u * c; if (r < R) a.out[((size_t)t * a.H + h) * R + r] = o[qi][c] * inv; }
        } else {
            float *dst = a.part + (((size_t)t * a.nsplit + split) * a.H + h) * (R + 2u);
#pragma unroll
            for (int c = 0; c < RCH; c++) { const uint32_t r = lane + 32u * c; if (r < R) dst[r] = o[qi][c]; }
            if (lane == 0) { dst[R] = m[qi]; dst[R + 1] = l[qi]; }
        }
    }
    if (a.nsplit == 1) return;
    // Key splits: every block has written partial (o, m, l) triples.  The block that draws the last ticket of its (query tile, head
    // group) sees all of them (fence before the ticket, fence after) and merges:
    //   out = sum_s e^{m_s - M} o_s / sum_s e^{m_s - M} l_s   over the splits that saw keys.
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
    if (!last_s || h >= a.H) return;
    __threadfence();
    const size_t stride = (size_t)a.H * (R + 2u);
    const uint32_t nact = min(a.nsplit, (tiles - tile_first + tps - 1u) / tps);      // splits that own key tiles; the others wrote nothing of weight
#pragma unroll
    for (int qi = 0; qi < QT; qi++) {
        if ((uint32_t)qi >= nq) continue;
        const uint32_t t = tq0 + qi;
        const float *base = a.part + ((size_t)t * a.nsplit * a.H + h) * (R + 2u);
        const bool live = lane < nact;
        const float ls = live ? __ldcg(base + lane * stride + R + 1u) : 0.0f;
        const float ms = (live && ls > 0.0f) ? __ldcg(base + lane * stride + R) : -INFINITY;
        float M = ms;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        if (a_sink) M = fmaxf(M, a_sink[h]);
        const float w = ls > 0.0f ? expf(ms - M) : 0.0f;
        float L = w * ls;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
        if (a_sink) L += expf(a_sink[h] - M);
        float acc[RCH];
#pragma unroll
        for (int c = 0; c < RCH; c++) acc[c] = 0.0f;
        // every one of these splits wrote its triple in this launch (zeros where no key was visible to this query), so the loop needs
        // no branch and its loads overlap
#pragma unroll 4
        for (uint32_t s = 0; s < nact; s++) {
            const float ws = __shfl_sync(0xffffffffu, w, s);
#pragma unroll
            for (int c = 0; c < RCH; c++) { const uint32_t r = lane + 32u * c; if (r < R) acc[c] = fmaf(ws, __ldcg(base + s * stride + r), acc[c]); }
        }
        const float inv = 1.0f / L;
#pragma unroll
        for (int c = 0; c < RCH; c++) { const uint32_t r = lane + 32u * c; if (r < R) a.out[((size_t)t * a.H + h) * R + r] = acc[c] * inv; }
    }
}

// ------------------------------------------------------------------------------------------------
// mixture of experts: routing
// ------------------------------------------------------------------------------------------------
// One block per token: router logits z_e = W_router[e] . h in fp32 (a warp per expert, lanes stride over the width), then the
// `top` largest (ties: the lower expert index first) and their weights = softmax over the chosen logits only; counts[e] += 1 per
// choice.  Dynamic shared memory: route_smem(NE, threads) bytes.
// mode 0: weights = softmax over the chosen logits; mode 1: weights = sigmoid of the chosen logits, taken as they are (they need not sum to 1);
// mode 2: scores = softmax over ALL experts, weights = the chosen experts' scores divided by their sum (+ 1e-20).
// extra: the router matrix carries that many more rows after the experts'; their logits go to extra_out [T][extra] and take no part
// in the choice (a gate of a shared expert, computed with the router's precision).  wrow (optional): the weights once more in
// expert-sorted row order, wrow[slot[t][j]] = wt[t][j], for a product that scales its rows.
struct RouteArgs { const float *h; const float *router; uint32_t *idx; float *wt; uint32_t *counts; uint32_t *off; uint32_t *fill; uint32_t *slot; uint32_t *rows; uint32_t T, NE, top, E;
                   uint32_t mode, extra; float *extra_out; float *wrow; };
// dynamic shared memory of k_route / k_route_small launched with `threads` threads (NE: rows of the router matrix, extra ones included)
inline size_t route_smem(uint32_t NE, uint32_t threads) { const uint32_t nw = threads / 32u; return ((size_t)NE + (size_t)NE * (nw > NE ? nw / NE : 1u)) * 4; }
// router logits of token t into z[NE].  The blockDim/32 warps are dealt out as `ns` slices per expert (ns = warps / NE, at least 1):
// a warp sums its slice of the row, the slices are added in order.  zp: NE * ns floats of scratch.
__device__ __forceinline__ uint32_t route_slices(uint32_t NE) { const uint32_t nw = blockDim.x >> 5; return nw > NE ? nw / NE : 1u; }
__device__ __forceinline__ void route_logits(const RouteArgs &a, uint32_t t, float *z, float *zp) {
    const uint32_t NL = a.NE + a.extra;          // rows of the router matrix
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nw = blockDim.x >> 5, ns = route_slices(NL);
    const float *h = a.h + (size_t)t * a.E;
    const bool vec = (a.E % 4u) == 0;
    const uint32_t per = ((a.E + ns - 1u) / ns + 3u) & ~3u;          // slice length, a multiple of 4
    for (uint32_t job = warp; job < NL * ns; job += nw) {
        const uint32_t e = job / ns, sl = job % ns;
        const uint32_t k0 = min(a.E, sl * per), k1 = min(a.E, k0 + per);
        const float *w = a.router + (size_t)e * a.E;
        float acc = 0.0f;
        if (vec) {
            for (uint32_t k = k0 + lane * 4u; k < k1; k += 128u) {
                const float4 hv = *reinterpret_cast<const float4 *>(h + k), wv = __ldg(reinterpret_cast<const float4 *>(w + k));
                acc = fmaf(hv.w, wv.w, fmaf(hv.z, wv.z, fmaf(hv.y, wv.y, fmaf(hv.x, wv.x, acc))));
            }
        } else {
            for (uint32_t k = k0 + lane; k < k1; k += 32u) acc = fmaf(h[k], w[k], acc);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) zp[job] = acc;
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < NL; e += blockDim.x) {
        float v = 0.0f;
        for (uint32_t sl = 0; sl < ns; sl++) v += zp[e * ns + sl];
        z[e] = v;
    }
}
// one thread: the `top` largest of z (ties: the lower index first; z is consumed) and the softmax over them
__device__ __forceinline__ void route_pick(const RouteArgs &a, uint32_t t, float *z) {
    uint32_t *idx = a.idx + (size_t)t * a.top; float *wt = a.wt + (size_t)t * a.top;
    float zmax = -INFINITY, zden = 0.0f;
    if (a.mode == 2u) {      // softmax over ALL experts: its maximum and denominator, before the choice consumes z
        for (uint32_t e = 0; e < a.NE; e++) zmax = fmaxf(zmax, z[e]);
        for (uint32_t e = 0; e < a.NE; e++) zden += expf(z[e] - zmax);
    }
    for (uint32_t j = 0; j < a.top; j++) {
        float best = -INFINITY; uint32_t bi = 0xffffffffu;
        for (uint32_t e = 0; e < a.NE; e++) {
            const float v = z[e];
            if (bi == 0xffffffffu || v > best) { best = v; bi = e; }
        }
        idx[j] = bi; wt[j] = best;
        z[bi] = -INFINITY;                 // taken (a logit that IS -inf can only tie with taken ones after all finite ones are gone)
    }
    for (uint32_t k = 0; k < a.extra; k++) a.extra_out[(size_t)t * a.extra + k] = z[a.NE + k];
    if (a.mode == 1u) { for (uint32_t j = 0; j < a.top; j++) wt[j] = sigmoidf_(wt[j]); return; }
    if (a.mode == 2u) {      // the chosen experts' scores, divided by their sum
        float s = 0.0f;
        for (uint32_t j = 0; j < a.top; j++) { wt[j] = expf(wt[j] - zmax) / zden; s += wt[j]; }
        for (uint32_t j = 0; j < a.top; j++) wt[j] /= s + 1e-20f;
        return;
    }
    const float mx = wt[0];
    float s = 0.0f;
    for (uint32_t j = 0; j < a.top; j++) { wt[j] = expf(wt[j] - mx); s += wt[j]; }
    for (uint32_t j = 0; j < a.top; j++) wt[j] /= s;
}
__global__ void __launch_bounds__(256) k_route(const RouteArgs a) {
    pdl_enter();
    extern __shared__ float z[];
    route_logits(a, blockIdx.x, z, z + a.NE + a.extra);
    __syncthreads();
    if (threadIdx.x) return;
    route_pick(a, blockIdx.x, z);
    for (uint32_t j = 0; j < a.top; j++) atomicAdd(a.counts + a.idx[(size_t)blockIdx.x * a.top + j], 1u);
}
// Short portions: routing and placement of all T tokens in one block of 1024 threads (the one block has the router matrix to itself,
// so every warp fetches).  Same outputs as k_route + k_route_place; the global counters are not touched.
__global__ void __launch_bounds__(1024) k_route_small(const RouteArgs a) {
    pdl_enter();
    extern __shared__ float z[];
    uint32_t *cur = reinterpret_cast<uint32_t *>(z);          // after the last token z is free
    for (uint32_t t = 0; t < a.T; t++) {
        route_logits(a, t, z, z + a.NE + a.extra);
        __syncthreads();
        if (threadIdx.x == 0) route_pick(a, t, z);
        __syncthreads();
    }
    if (threadIdx.x) return;
    const uint32_t n = a.T * a.top;
    for (uint32_t e = 0; e < a.NE; e++) cur[e] = 0;
    for (uint32_t i = 0; i < n; i++) cur[a.idx[i]]++;
    uint32_t s = 0;
    for (uint32_t e = 0; e < a.NE; e++) { const uint32_t c = cur[e]; a.off[e] = s; cur[e] = s; s += c; }
    a.off[a.NE] = s;
    for (uint32_t i = 0; i < n; i++) { const uint32_t sl = cur[a.idx[i]]++; a.slot[i] = sl; a.rows[sl] = i / a.top; if (a.wrow) a.wrow[sl] = a.wt[i]; }
}
// One block: off[e] = rows before expert e (off[NE] = total), counters cleared for the next use; then slot[t][j] = the row of
// (token t, choice j) in the expert-sorted order and rows[slot] = t
__global__ void __launch_bounds__(1024) k_route_place(const RouteArgs a) {
    pdl_enter();
    if (threadIdx.x == 0) {
        uint32_t s = 0;
        for (uint32_t e = 0; e < a.NE; e++) { a.off[e] = s; s += a.counts[e]; a.counts[e] = 0; a.fill[e] = 0; }
        a.off[a.NE] = s;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < a.T * a.top; i += blockDim.x) {
        const uint32_t e = a.idx[i];
        const uint32_t s = a.off[e] + atomicAdd(a.fill + e, 1u);
        a.slot[i] = s; a.rows[s] = i / a.top;
        if (a.wrow) a.wrow[s] = a.wt[i];
    }
}

// x[t] += d[t] + ( sum_j wt[t][j] * eo[slot[t][j]]  (+ shared[t]) ),  the sum in the order of the choices; keep (optional) gets x
struct CombineArgs { float *x; const float *d; const float *eo; const uint32_t *slot; const float *wt; const float *shared; float *keep; uint32_t T, E, top; };
__global__ void k_combine(const CombineArgs a) {
    pdl_enter();
    const size_t total = (size_t)a.T * a.E;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t t = (uint32_t)(i / a.E), c = (uint32_t)(i % a.E);
        float delta = a.d[i];
        if (a.eo) {
            float f = 0.0f;
            for (uint32_t j = 0; j < a.top; j++) f = fmaf(a.wt[(size_t)t * a.top + j], a.eo[(size_t)a.slot[(size_t)t * a.top + j] * a.E + c], f);
            if (a.shared) f += a.shared[i];
            delta += f;
        }
        const float v = a.x[i] + delta;
        a.x[i] = v;
        if (a.keep) a.keep[i] = v;
    }
}

// scalar-gain RMS norm of the rows whose logits are asked for: out[i] = x[want[i]] / rms * g
// (vec: the gain is a vector stored around zero, out = x / rms * (1 + g[i]))
__global__ void __launch_bounds__(256) k_final_norm(const float *__restrict__ x, const uint32_t *__restrict__ want, const float *__restrict__ g,
                                                    float *__restrict__ out, uint32_t E, float eps, uint32_t vec) {
    pdl_enter();
    __shared__ float red[32];
    const float *xt = x + (size_t)want[blockIdx.x] * E;
    float s = 0.0f;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) s = fmaf(xt[i], xt[i], s);
    s = block_sum(s, red);
    const float rinv = 1.0f / sqrtf(s / (float)E + eps) * 1.0f;
    const float gv = vec ? 0.0f : *g;
    for (uint32_t i = threadIdx.x; i < E; i += blockDim.x) out[(size_t)blockIdx.x * E + i] = xt[i] * rinv * (vec ? 1.0f + g[i] : gv);
}

// greedy choice with the repetition penalty of the generation hosts: logits of ids seen before are divided (positive) or multiplied
// (negative) by `penalty`; the lowest index wins ties.  One block.  ids[pos + 1] receives the choice unless that place is still
// inside the prompt (pos + 1 < n_prompt); pos is read from (and advanced in) *pos_ptr when given.  penalised (optional) receives the logits after the penalty, for the sampler.
struct PickArgs { float *logits; const uint8_t *seen; uint8_t *seen_rw; uint32_t *ids; uint32_t *next; uint32_t V, pos, n_prompt; float penalty; uint32_t advance; uint32_t *pos_ptr; };
__global__ void __launch_bounds__(1024) k_pick(const PickArgs a) {
    pdl_enter();
    __shared__ float bv[32]; __shared__ uint32_t bi[32];
    float best = -INFINITY; uint32_t idx = 0xffffffffu;
    for (uint32_t i = threadIdx.x; i < a.V; i += blockDim.x) {
        float v = a.logits[i];
        if (a.penalty != 1.0f && a.seen[i]) { v = v > 0.0f ? v / a.penalty : v * a.penalty; a.logits[i] = v; }
        if (v > best || idx == 0xffffffffu) { best = v; idx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o); const uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi != 0xffffffffu && (idx == 0xffffffffu || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
    }
    if ((threadIdx.x & 31u) == 0) { bv[threadIdx.x >> 5] = best; bi[threadIdx.x >> 5] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < (blockDim.x >> 5); w++)
            if (bi[w] != 0xffffffffu && (bi[0] == 0xffffffffu || bv[w] > bv[0] || (bv[w] == bv[0] && bi[w] < bi[0]))) { bv[0] = bv[w]; bi[0] = bi[w]; }
        uint32_t nxt = bi[0];
        if (a.advance) {      // the device loop: pos lives on the device and moves on with the choice
            const uint32_t pos = a.pos_ptr ? *a.pos_ptr : a.pos;
            a.seen_rw[a.ids[pos]] = 1;
            if (pos + 1 < a.n_prompt) nxt = a.ids[pos + 1]; else a.ids[pos + 1] = nxt;
            if (a.pos_ptr) *a.pos_ptr = pos + 1;
        }
        *a.next = nxt;
    }
}
__global__ void k_mark(uint8_t *seen, const uint32_t *ids, uint32_t n) {
    pdl_enter();
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) seen[ids[i]] = 1;
}

}  // namespace lm
}  // namespace nb

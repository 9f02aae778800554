// Hyper-connections: a residual of S parallel streams x_1 .. x_S (a token's row holds them side by side, [S * D],
// 32-bit) in place of the single residual sum.  A sublayer reads ONE mix of the streams and writes to all of them:
//
//   read    u = sum_s in[s] x_s                       then a norm of u feeds the sublayer
//   write   x_t <- sum_s mix[s][t] x_s + out[t] * y   for all t at once, from the old streams; y the sublayer's result
//
// hyper_step does, per token and in one pass over its row: the write of the sublayer that has just run (if `y` or
// `pairs` is given; with `pairs` the result is y, if given, plus the weighted sum over the token's `top` chosen experts,
// pairs[token * top + k] * pair_w[token * top + k] in the order of k: a routed feed-forward's last step), then the
// read of the next sublayer from the new streams and its norm (if `h` is given): LayerNorm with weight and bias, (u - mean) / sqrt(var + eps) * gamma + beta with the variance as the mean of the squared deviations, or an
// RMS norm (no centring, no bias) when beta is null.  With `in` null the read is the plain sum of the streams (what the
// model's last norm sees).  `rows` gathers the tokens that are read; a write then happens on the way for those tokens only
// (y and pairs are indexed by token) and is not stored: the streams of a step's last layer, of which only the wanted
// tokens' sum is read.  Everything is 32-bit; h is
// rounded to the activation dtype.  One CTA per token; u is kept in shared memory; the sums over s run in stream
// order, so a token's result does not depend on the batch.
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 8;

// NS: the number of streams when it is 1 .. 4 (the sums over streams unroll to exactly that many terms and the kernel
// keeps few registers), or MAX_STREAMS for any count up to that (terms past S are skipped at run time).
template <typename TOut, int NS>
__global__ void __launch_bounds__(256)
hyper_step_kernel(float* x, const float* y, long long ldy, const float* __restrict__ mix, const float* __restrict__ outw,
                  const float* __restrict__ inw, const float* __restrict__ gamma, const float* __restrict__ beta, float eps,
                  const int* __restrict__ rows, TOut* h, long long ldh, float* sum_out, const float* pairs, const float* pair_w,
                  int top, int S, int D) {
    extern __shared__ float u[];            // [D]
    __shared__ float scratch[33];
    __shared__ float s_mix[MAX_STREAMS * MAX_STREAMS], s_out[MAX_STREAMS], s_in[MAX_STREAMS];
    const int tid = threadIdx.x;
    if (tid < S * S) s_mix[tid] = mix ? mix[tid] : 0.f;          // weights: nothing of the step writes them
    if (tid < S) { s_out[tid] = outw ? outw[tid] : 0.f; s_in[tid] = inw ? inw[tid] : 1.f; }
    pdl_wait();
    pdl_launch();
    __syncthreads();
    const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
    float* xr = x + r * (size_t)S * D;
    const float* yr = y ? y + r * ldy : nullptr;
    const float* pr = pairs ? pairs + r * top * D : nullptr;
    const float* pw = pairs ? pair_w + r * top : nullptr;
    const bool writes = yr != nullptr || pr != nullptr;
    const bool reads = h != nullptr || sum_out != nullptr;
    float part = 0.f;
    for (int d = tid; d < D; d += blockDim.x) {
        float xs[NS];
#pragma unroll
        for (int s = 0; s < NS; ++s) xs[s] = s < S ? xr[(size_t)s * D + d] : 0.f;
        if (writes) {
            float yv = yr ? yr[d] : 0.f;
            for (int k = 0; k < top; ++k) yv = fmaf(pw[k], pr[(size_t)k * D + d], yv);
            float nx[NS];
#pragma unroll
            for (int t = 0; t < NS; ++t) {
                if (t < S) {
                    float a = 0.f;
#pragma unroll
                    for (int s = 0; s < NS; ++s)
                        if (s < S) a = fmaf(s_mix[s * S + t], xs[s], a);
                    nx[t] = fmaf(s_out[t], yv, a);
                }
            }
#pragma unroll
            for (int t = 0; t < NS; ++t)
                if (t < S) {
                    xs[t] = nx[t];
                    if (!rows) xr[(size_t)t * D + d] = nx[t];    // gathered rows are read only: the same row may be asked for twice
                }
        }
        if (reads) {
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < NS; ++s)
                if (s < S) a = fmaf(s_in[s], xs[s], a);
            u[d] = a;
            part += a;
        }
    }
    if (!reads) return;
    if (sum_out)
        for (int d = tid; d < D; d += blockDim.x) sum_out[(size_t)blockIdx.x * D + d] = u[d];    // each thread re-reads its own entries
    if (!h) return;
    float mean = 0.f;
    if (beta) mean = block_sum(part, scratch) / (float)D;
    float sq = 0.f;
    for (int d = tid; d < D; d += blockDim.x) { const float c = u[d] - mean; sq = fmaf(c, c, sq); }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)D + eps);
    TOut* hr = h + (size_t)blockIdx.x * ldh;
    for (int d = tid; d < D; d += blockDim.x) hr[d] = from_f32<TOut>((u[d] - mean) * rstd * gamma[d] + (beta ? beta[d] : 0.f));
}

}  // namespace

MLLM_EXPORT int mllm_hyper_max_streams() { return MAX_STREAMS; }

// x [., S * D] 32-bit.  y [R, D] 32-bit with mix [S * S] ([from][to]) and outw [S], or all null (no write).
// h [R, D] (dtype) with gamma [D], beta [D] or null (RMS norm), inw [S] or null (plain sum), or null (no read);
// sum_out [R, D] 32-bit or null: the read before its norm.  rows [R] or null (then y and pairs are indexed by the token
// rows[r], and the new streams are not stored).  pairs [. * top, D] with pair_w [. * top]
// (32-bit), or null: the chosen experts' results and weights, summed into the written result.
MLLM_EXPORT int mllm_hyper_step(float* x, const float* y, long long ldy, const float* mix, const float* outw, const float* inw,
                                const float* gamma, const float* beta, float eps, const int* rows, void* h, long long ldh,
                                float* sum_out, const float* pairs, const float* pair_w, int top, int R, int S, int D, int dtype,
                                cudaStream_t stream) {
    if (R <= 0) return 0;
    if (S <= 0 || S > MAX_STREAMS || D <= 0) return mllm_fail(1, "hyper_step: %d streams of width %d (at most %d streams)", S, D, MAX_STREAMS);
    if (!pairs) top = 0;
    if (pairs && (!pair_w || top <= 0)) return mllm_fail(1, "hyper_step: the experts' results need their weights and a count");
    if ((y || pairs) && (!mix || !outw)) return mllm_fail(1, "hyper_step: a write needs the mixing matrix and the output weights");
    if (h && !gamma) return mllm_fail(1, "hyper_step: a norm needs its weight");
    if (!y && !pairs && !h && !sum_out) return 0;
    const size_t smem = sizeof(float) * (size_t)D;
    if (smem > 200 * 1024) return mllm_fail(1, "hyper_step: width %d does not fit shared memory", D);
    if (dtype != MLLM_F32 && dtype != MLLM_BF16) return mllm_fail(1, "hyper_step: unknown dtype code %d", dtype);
#define HYPER_LAUNCH(TOUT, NS)                                                                                              \
    do {                                                                                                                    \
        if (smem > 48 * 1024)                                                                                               \
            MLLM_CUDA(cudaFuncSetAttribute(hyper_step_kernel<TOUT, NS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MLLM_CUDA(mllm_launch(hyper_step_kernel<TOUT, NS>, dim3(R), dim3(256), smem, stream, true, x, y, ldy, mix, outw, inw, \
                              gamma, beta, eps, rows, (TOUT*)h, ldh, sum_out, pairs, pair_w, top, S, D));                    \
    } while (0)
#define HYPER_BY_STREAMS(TOUT)                                                                                              \
    switch (S) {                                                                                                            \
        case 1: HYPER_LAUNCH(TOUT, 1); break;                                                                               \
        case 2: HYPER_LAUNCH(TOUT, 2); break;                                                                               \
        case 3: HYPER_LAUNCH(TOUT, 3); break;                                                                               \
        case 4: HYPER_LAUNCH(TOUT, 4); break;                                                                               \
        default: HYPER_LAUNCH(TOUT, MAX_STREAMS); break;                                                                    \
    }
    if (dtype == MLLM_F32) {
        HYPER_BY_STREAMS(float);
    } else {
        HYPER_BY_STREAMS(__nv_bfloat16);
    }
#undef HYPER_BY_STREAMS
#undef HYPER_LAUNCH
    return 0;
}

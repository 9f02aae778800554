// A linear recurrence with a matrix state per head, a decay per key channel that depends on the token, and a bonus for
// the current token (RWKV-style time mixing).  Per head, with r_t, k_t, v_t rows of n entries and S [n, n] zero at the
// start of a sequence:
//   w_t = exp(-exp(W2 tanh(l_t) + w0))                 l_t: a low-rank projection of the token (R entries), W2 [n, R]
//   o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t          the bonus u counts for the current token only
//   S_t = diag(w_t) S_(t-1) + k_t v_t^T
//   y_t = o_t / sqrt(mean(o_t^2) + eps) * g * silu(z_t)   g: a weight per channel, z: the gate's projection
// The inputs of the five projections are mixes of a token's row with the row before it: m_s = h + (h' - h) * mu_s, h'
// the previous token's h (zeros before the first token); the last row of a step is kept in the request's state next
// to S, so that the next step finds it.  State, decay (tanh, both exponentials), the update, o, the norm and the gate
// are 32-bit whatever the dtype of the projections.
//
// Five kernels.  `step`: steps of single tokens in one launch (decay, update, output, norm and gate; described where it
// stands).  The other four take steps that carry prompt portions.  `shift`: the mixes of every token (one CTA per token).  `decay`: the decays of every token and channel,
// off the recurrence's sequential path.  `scan`: a CTA takes 32 columns of one
// (request, head)'s state; thread (lane, g) keeps rows g*WR .. g*WR+WR-1 of column lane in registers for the whole walk,
// tokens come CH at a time (r, k, the decays and v staged in shared memory, the next chunk's fetched into registers
// meanwhile), the row groups' partial outputs meet in
// group order; every element of the state is a recurrence of its own, so the state after n tokens is the same bits
// however the tokens were cut into steps.  `finish`: one warp per (token, head): the unit norm, the weight and the gate.
#include "common.cuh"

namespace {

constexpr int WKV_CH = 16;          // tokens per chunk of the scan

template <typename T>
__global__ void __launch_bounds__(256)
wkv_shift_kernel(const T* h, long long ldh, const float* __restrict__ mu, const float* state, long long state_stride,
                 long long prev_off, const int* __restrict__ token_seq, const int* __restrict__ cu_q,
                 const int* __restrict__ slots, const int* __restrict__ positions, T* __restrict__ mixes, int Tn, int D, int NS) {
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x;
    const int seq = token_seq[t];
    const bool inside = t > cu_q[seq];                          // the row before is a token of this step
    const bool has_state = positions[t] > 0;                    // else: the first token of a sequence sees zeros
    const T* cur = h + (size_t)t * ldh;
    const T* before = h + (size_t)(t - (inside ? 1 : 0)) * ldh;
    const float* kept = state + (size_t)slots[seq] * state_stride + prev_off;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float x = to_f32(cur[d]);
        const float p = inside ? to_f32(before[d]) : (has_state ? kept[d] : 0.f);
        const float diff = p - x;
        for (int s = 0; s < NS; ++s)
            mixes[((size_t)s * Tn + t) * D + d] = from_f32<T>(fmaf(diff, mu[(size_t)s * D + d], x));
    }
}

// w[t][c] = exp(-exp(w0[c] + sum_q W2[c][q] tanh(low[t][q]))): a CTA takes 16 tokens and 64 channels; the tokens' tanh
// values and (64 ranks at a time) the channels' rows of W2 are staged in shared memory with loads along the rows, a
// thread keeps one channel's sums for four tokens.  Every token's sum runs over q in the same order, whatever else is
// in the step.
constexpr int DEC_TOK = 16, DEC_CH = 64, DEC_Q = 64;

template <typename T>
__global__ void __launch_bounds__(256)
wkv_decay_kernel(const T* low, long long l_stride, const T* __restrict__ W2, const float* __restrict__ w0, float* __restrict__ w,
                 long long w_stride, int Tn, int N, int R) {
    extern __shared__ float tl[];           // [DEC_TOK][R], then the tile of W2 [DEC_Q][DEC_CH + 1]
    float* wt = tl + DEC_TOK * R;
    const int ch0 = blockIdx.y * DEC_CH;
    const int chl = threadIdx.x & (DEC_CH - 1), tg = threadIdx.x / DEC_CH;     // this thread's channel; tokens tg, tg + 4, ...
    const int ch = ch0 + chl;
    auto stage_w = [&](int q0) {            // weights: may be read before the kernel before this one has ended
        for (int idx = threadIdx.x; idx < DEC_CH * DEC_Q; idx += blockDim.x) {
            const int c = idx / DEC_Q, q = idx % DEC_Q;
            wt[q * (DEC_CH + 1) + c] = (ch0 + c < N && q0 + q < R) ? to_f32(W2[(size_t)(ch0 + c) * R + q0 + q]) : 0.f;
        }
    };
    stage_w(0);
    pdl_wait();
    pdl_launch();
    const int t0 = blockIdx.x * DEC_TOK, nt = min(DEC_TOK, Tn - t0);
    for (int idx = threadIdx.x; idx < DEC_TOK * R; idx += blockDim.x) {
        const int c = idx / R, q = idx % R;
        tl[idx] = c < nt ? tanhf(to_f32(low[(size_t)(t0 + c) * l_stride + q])) : 0.f;
    }
    float acc[DEC_TOK / 4];
    const float b = ch < N ? w0[ch] : 0.f;
#pragma unroll
    for (int u = 0; u < DEC_TOK / 4; ++u) acc[u] = b;
    for (int q0 = 0; q0 < R; q0 += DEC_Q) {
        if (q0 > 0) {
            __syncthreads();                // the tile before is no longer read
            stage_w(q0);
        }
        __syncthreads();
        const int nq = min(DEC_Q, R - q0);
        for (int q = 0; q < nq; ++q) {
            const float wv = wt[q * (DEC_CH + 1) + chl];
#pragma unroll
            for (int u = 0; u < DEC_TOK / 4; ++u) acc[u] = fmaf(wv, tl[(tg + 4 * u) * R + q0 + q], acc[u]);
        }
    }
    if (ch >= N) return;
#pragma unroll
    for (int u = 0; u < DEC_TOK / 4; ++u) {
        const int c = tg + 4 * u;
        if (c < nt) w[(size_t)(t0 + c) * w_stride + ch] = expf(-expf(acc[u]));
    }
}

struct WkvArgs {
    const int* cu_q;        // [S+1] first flat token of every request of the step
    const int* slots;       // [S] state slot of every request
    const float* u;         // [Hr*n]
    float* state;           // [slots][state_stride]: S of every head [Hr][n][n], then the last row of h at prev_off
    long long state_stride, prev_off;
    long long r_stride, k_stride, v_stride, w_stride, o_stride, h_stride;
    int Hr, n, D, write_state;
};

// grid (requests, heads, ceil(n / COLS)); block (COLS, G), G = ceil(n / WR).  o [T][Hr*n] float.  COLS, the columns of the
// state a CTA takes, is 32, or 16 when that is what fills the SMs (few requests and heads).  The next chunk's inputs
// are fetched into registers while the current chunk is walked, so the walk never waits for global memory.
template <typename T, int WR, int COLS>
__global__ void __launch_bounds__(COLS * 32)
wkv_scan_kernel(const T* r, const T* k, const T* v, const float* w, const T* h, float* __restrict__ o, WkvArgs a) {
    extern __shared__ __align__(16) float sm[];
    constexpr int PF = WKV_CH * WR / COLS;      // elements of r (and of k, of w) a thread fetches per chunk
    constexpr int PFV = 2;                    // elements of v a thread fetches ahead (WKV_CH / G of them; with fewer than 8
                                              // row groups, i.e. tiny heads, v is staged directly instead)
    const int n = a.n, G = blockDim.y, np = G * WR;    // rows padded to a multiple of WR: the padding has r = k = 0, w = 1
    float* rs = sm;                           // [CH][np]
    float* ks = rs + WKV_CH * np;             // [CH][np]
    float* ws = ks + WKV_CH * np;             // [CH][np]
    float* vs = ws + WKV_CH * np;             // [CH][COLS]
    float* os = vs + WKV_CH * COLS;       // [G][CH][COLS]
    pdl_wait();
    pdl_launch();
    const int seq = blockIdx.x, hd = blockIdx.y, j0 = blockIdx.z * COLS;
    const int lane = threadIdx.x, g = threadIdx.y, tid = g * COLS + lane, nthreads = G * COLS;
    const int t0 = a.cu_q[seq], t1 = a.cu_q[seq + 1];
    if (t1 <= t0) return;
    const int slot = a.slots[seq];
    const int j = j0 + lane;
    const bool col = j < n;
    float* sp = a.state + (size_t)slot * a.state_stride + ((size_t)hd * n) * n + j;
    float s[WR], uu[WR];
#pragma unroll
    for (int i = 0; i < WR; ++i) {
        const int row = g * WR + i;
        s[i] = (col && row < n) ? sp[(size_t)row * n] : 0.f;
        uu[i] = row < n ? a.u[hd * n + row] : 0.f;
    }
    // the row that the next step's first token mixes with: the last row of h of this step
    if (a.write_state && hd == 0 && blockIdx.z == 0) {
        float* kept = a.state + (size_t)slot * a.state_stride + a.prev_off;
        const T* last = h + (size_t)(t1 - 1) * a.h_stride;
        for (int d = tid; d < a.D; d += nthreads) kept[d] = to_f32(last[d]);
    }
    // which elements of a chunk this thread fetches: the same in every chunk
    int e_c[PF], e_i[PF];
#pragma unroll
    for (int x = 0; x < PF; ++x) {
        const int idx = tid + x * nthreads;
        e_c[x] = idx / np;
        e_i[x] = idx % np;
    }
    const int vcount = (WKV_CH * COLS + nthreads - 1) / nthreads;
    const bool v_ahead = vcount <= PFV;
    float pr[PF], pk[PF], pw[PF], pv[PFV];
    auto fetch = [&](int c0) {
        const int nc = min(WKV_CH, t1 - c0);
#pragma unroll
        for (int x = 0; x < PF; ++x) {
            pr[x] = 0.f; pk[x] = 0.f; pw[x] = 1.f;
            if (e_c[x] < nc && e_i[x] < n) {
                const size_t t = (size_t)(c0 + e_c[x]);
                const size_t cix = (size_t)hd * n + e_i[x];
                pr[x] = to_f32(r[t * a.r_stride + cix]);
                pk[x] = to_f32(k[t * a.k_stride + cix]);
                pw[x] = w[t * a.w_stride + cix];
            }
        }
#pragma unroll
        for (int x = 0; x < PFV; ++x) {
            pv[x] = 0.f;
            if (v_ahead && x < vcount) {
                const int idx = tid + x * nthreads, c = idx / COLS, d = idx % COLS;
                if (idx < WKV_CH * COLS && c < nc && j0 + d < n)
                    pv[x] = to_f32(v[(size_t)(c0 + c) * a.v_stride + (size_t)hd * n + j0 + d]);
            }
        }
    };
    fetch(t0);
    for (int c0 = t0; c0 < t1; c0 += WKV_CH) {
        const int nc = min(WKV_CH, t1 - c0);
        __syncthreads();                      // the chunk before is no longer read
#pragma unroll
        for (int x = 0; x < PF; ++x) {
            const int idx = tid + x * nthreads;
            rs[idx] = pr[x];
            ks[idx] = pk[x];
            ws[idx] = pw[x];
        }
        if (v_ahead) {
#pragma unroll
            for (int x = 0; x < PFV; ++x) {
                const int idx = tid + x * nthreads;
                if (x < vcount && idx < WKV_CH * COLS) vs[idx] = pv[x];
            }
        } else {
            for (int idx = tid; idx < WKV_CH * COLS; idx += nthreads) {
                const int c = idx / COLS, d = idx % COLS;
                vs[idx] = (c < nc && j0 + d < n) ? to_f32(v[(size_t)(c0 + c) * a.v_stride + (size_t)hd * n + j0 + d]) : 0.f;
            }
        }
        __syncthreads();
        if (c0 + WKV_CH < t1) fetch(c0 + WKV_CH);
        for (int c = 0; c < nc; ++c) {
            const float vj = vs[c * COLS + lane];
            const float* rr = rs + c * np + g * WR;
            const float* kk = ks + c * np + g * WR;
            const float* ww = ws + c * np + g * WR;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < WR; ++i) {
                const float kv = kk[i] * vj;
                acc = fmaf(rr[i], fmaf(uu[i], kv, s[i]), acc);
                s[i] = fmaf(ww[i], s[i], kv);
            }
            os[(g * WKV_CH + c) * COLS + lane] = acc;
        }
        __syncthreads();
        for (int idx = tid; idx < nc * COLS; idx += nthreads) {       // the row groups meet in group order
            const int c = idx / COLS, d = idx % COLS;
            if (j0 + d >= n) continue;
            float acc = os[c * COLS + d];
            for (int gg = 1; gg < G; ++gg) acc += os[(gg * WKV_CH + c) * COLS + d];
            o[(size_t)(c0 + c) * a.o_stride + (size_t)hd * n + j0 + d] = acc;
        }
    }
    if (a.write_state && col) {
#pragma unroll
        for (int i = 0; i < WR; ++i)
            if (g * WR + i < n) sp[(size_t)(g * WR + i) * n] = s[i];
    }
}

// one warp per (token, head): y = o / sqrt(mean(o^2) + eps) * weight * silu(z)
template <typename T>
__global__ void __launch_bounds__(128)
wkv_finish_kernel(const float* o, long long o_stride, const T* z, long long z_stride, const float* __restrict__ weight,
                  T* __restrict__ y, long long y_stride, int Tn, int Hr, int n, float eps) {
    pdl_wait();
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * 4 + warp;
    if (gw >= (long long)Tn * Hr) return;
    const int t = (int)(gw / Hr), hd = (int)(gw % Hr);
    const float* orow = o + (size_t)t * o_stride + (size_t)hd * n;
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) { const float x = orow[d]; ss = fmaf(x, x, ss); }
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
    for (int d = lane; d < n; d += 32) {
        const float zz = to_f32(z[(size_t)t * z_stride + (size_t)hd * n + d]);
        y[(size_t)t * y_stride + (size_t)hd * n + d] = from_f32<T>(orow[d] * inv * weight[hd * n + d] * (zz / (1.0f + expf(-zz))));
    }
}

// Steps of single tokens: the decay, the state's update, the output, its unit norm, the weight and the gate in one
// launch.  One CTA per (request, head); thread (column j, row group g) keeps RK rows of column j of the state in
// registers.  The head's rows of W2 come into shared memory with loads along the rows before the kernel waits for its
// predecessor (they are weights).  The decays are the same bits as the decay pass's (one sum per channel over q in
// order), and every state element takes the same update as in the scan, so the state is the same bits whichever kernel
// took a token.  A request's tokens (one in a decode step) are walked in order.
template <typename T, int RK>
__global__ void __launch_bounds__(1024)
wkv_step_kernel(const T* r, const T* k, const T* v, const T* low, const T* __restrict__ W2, const float* __restrict__ w0,
                const T* z, const float* __restrict__ weight, const T* h, T* __restrict__ y, long long l_stride,
                long long z_stride, long long y_stride, int R, int evp, float eps, WkvArgs a) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float scratch[33];
    const int n = a.n, tid = threadIdx.x, nthreads = blockDim.x;
    const int G = nthreads / evp, j = tid % evp, g = tid / evp;
    float* w2s = sm;                          // [n][R + 1]
    float* tl = w2s + n * (R + 1);            // [R]
    float* rs = tl + R;                       // [n]
    float* ks = rs + n;                       // [n]
    float* ws = ks + n;                       // [n]
    float* vs = ws + n;                       // [evp]
    float* os = vs + evp;                     // [G][evp]
    const int seq = blockIdx.x, hd = blockIdx.y;
    for (int idx = tid; idx < n * R; idx += nthreads) {
        const int i = idx / R, q = idx % R;
        w2s[i * (R + 1) + q] = to_f32(W2[((size_t)hd * n + i) * R + q]);
    }
    pdl_wait();
    pdl_launch();
    const int t0 = a.cu_q[seq], t1 = a.cu_q[seq + 1];
    if (t1 <= t0) return;
    const int slot = a.slots[seq];
    const bool col = j < n;
    float* sp = a.state + (size_t)slot * a.state_stride + ((size_t)hd * n) * n + j;
    float s[RK], uu[RK];
#pragma unroll
    for (int i = 0; i < RK; ++i) {
        const int row = g * RK + i;
        s[i] = (col && row < n) ? sp[(size_t)row * n] : 0.f;
        uu[i] = row < n ? a.u[hd * n + row] : 0.f;
    }
    if (a.write_state && hd == 0) {
        float* kept = a.state + (size_t)slot * a.state_stride + a.prev_off;
        const T* last = h + (size_t)(t1 - 1) * a.h_stride;
        for (int d = tid; d < a.D; d += nthreads) kept[d] = to_f32(last[d]);
    }
    for (int t = t0; t < t1; ++t) {
        __syncthreads();                      // the token before is no longer read; the weights are staged
        for (int q = tid; q < R; q += nthreads) tl[q] = tanhf(to_f32(low[(size_t)t * l_stride + q]));
        for (int i = tid; i < n; i += nthreads) {
            rs[i] = to_f32(r[(size_t)t * a.r_stride + (size_t)hd * n + i]);
            ks[i] = to_f32(k[(size_t)t * a.k_stride + (size_t)hd * n + i]);
        }
        for (int d = tid; d < evp; d += nthreads) vs[d] = d < n ? to_f32(v[(size_t)t * a.v_stride + (size_t)hd * n + d]) : 0.f;
        __syncthreads();
        for (int i = tid; i < n; i += nthreads) {
            float acc = w0[hd * n + i];
            const float* wr = w2s + i * (R + 1);
            for (int q = 0; q < R; ++q) acc = fmaf(wr[q], tl[q], acc);
            ws[i] = expf(-expf(acc));
        }
        __syncthreads();
        const float vj = vs[j];
        float acc = 0.f;
#pragma unroll
        for (int i = 0; i < RK; ++i) {
            const int row = g * RK + i;
            if (row < n) {
                const float kv = ks[row] * vj;
                acc = fmaf(rs[row], fmaf(uu[i], kv, s[i]), acc);
                s[i] = fmaf(ws[row], s[i], kv);
            }
        }
        os[g * evp + j] = acc;
        __syncthreads();
        float o = 0.f;
        if (g == 0 && col) {                  // the row groups meet in group order
            o = os[j];
            for (int gg = 1; gg < G; ++gg) o += os[gg * evp + j];
        }
        const float inv = 1.0f / sqrtf(block_sum(o * o, scratch) / (float)n + eps);
        if (g == 0 && col) {
            const float zz = to_f32(z[(size_t)t * z_stride + (size_t)hd * n + j]);
            y[(size_t)t * y_stride + (size_t)hd * n + j] = from_f32<T>(o * inv * weight[hd * n + j] * (zz / (1.0f + expf(-zz))));
        }
    }
    if (a.write_state && col) {
#pragma unroll
        for (int i = 0; i < RK; ++i)
            if (g * RK + i < n) sp[(size_t)(g * RK + i) * n] = s[i];
    }
}

}  // namespace

MLLM_EXPORT int mllm_wkv_max_dim() { return 256; }

// mixes [NS][T][D] = h + (row before - h) * mu[s]; the row before a step's first token of a request is the one kept in
// its state (zeros at position 0).
MLLM_EXPORT int mllm_wkv_shift(const void* h, long long ldh, const float* mu, const float* state, long long state_stride,
                               long long prev_off, const int* token_seq, const int* cu_q, const int* slots,
                               const int* positions, void* mixes, int T, int D, int NS, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (D <= 0 || NS <= 0) return mllm_fail(1, "wkv_shift: width %d, %d mixes", D, NS);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(wkv_shift_kernel<float>, dim3(T), dim3(256), 0, stream, true, (const float*)h, ldh, mu, state,
                              state_stride, prev_off, token_seq, cu_q, slots, positions, (float*)mixes, T, D, NS));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(wkv_shift_kernel<__nv_bfloat16>, dim3(T), dim3(256), 0, stream, true, (const __nv_bfloat16*)h, ldh,
                              mu, state, state_stride, prev_off, token_seq, cu_q, slots, positions, (__nv_bfloat16*)mixes, T, D, NS));
    else
        return mllm_fail(1, "wkv_shift: unknown dtype code %d", dtype);
    return 0;
}

// low [T, R], W2 [N, R] in `dtype`; w0 [N] float; w [T, N] float = exp(-exp(W2 tanh(low) + w0)).
MLLM_EXPORT int mllm_wkv_decay(const void* low, long long l_stride, const void* W2, const float* w0, float* w, long long w_stride,
                               int T, int N, int R, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (N <= 0 || R <= 0) return mllm_fail(1, "wkv_decay: %d channels, rank %d", N, R);
    const size_t smem = sizeof(float) * ((size_t)DEC_TOK * R + DEC_Q * (DEC_CH + 1));
    if (smem > 96 * 1024) return mllm_fail(1, "wkv_decay: rank %d does not fit shared memory", R);
    const dim3 grid((T + DEC_TOK - 1) / DEC_TOK, (N + DEC_CH - 1) / DEC_CH);
    if (grid.y > 65535) return mllm_fail(1, "wkv_decay: too many channels");
    if (dtype == MLLM_F32) {
        if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(wkv_decay_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MLLM_CUDA(mllm_launch(wkv_decay_kernel<float>, grid, dim3(256), smem, stream, true, (const float*)low, l_stride,
                              (const float*)W2, w0, w, w_stride, T, N, R));
    } else if (dtype == MLLM_BF16) {
        if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(wkv_decay_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MLLM_CUDA(mllm_launch(wkv_decay_kernel<__nv_bfloat16>, grid, dim3(256), smem, stream, true, (const __nv_bfloat16*)low,
                              l_stride, (const __nv_bfloat16*)W2, w0, w, w_stride, T, N, R));
    } else {
        return mllm_fail(1, "wkv_decay: unknown dtype code %d", dtype);
    }
    return 0;
}

// r, k, v [T, Hr*n] in `dtype`; w [T, Hr*n] float (the decays); u [Hr*n] float; h [T, D] (its last row of every request is
// kept); state [slots][state_stride] float with S at 0 and the kept row at prev_off; o [T, Hr*n] float.  want_cols: the
// columns of a state per CTA, 16 or 32, or 0 for the rule below (outputs and states are the same bits either way).
MLLM_EXPORT int mllm_wkv_scan(const void* r, long long r_stride, const void* k, long long k_stride, const void* v,
                              long long v_stride, const float* w, long long w_stride, const float* u, const void* h,
                              long long h_stride, float* state, long long state_stride, long long prev_off, const int* cu_q,
                              const int* slots, float* o, long long o_stride, int S, int Hr, int n, int D, int write_state,
                              int want_cols, int dtype, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (Hr <= 0 || n <= 0 || n > 256) return mllm_fail(1, "wkv_scan: %d heads of %d", Hr, n);
    if (Hr > 65535) return mllm_fail(1, "wkv_scan: grid of %d x %d", S, Hr);
    const int WR = n <= 64 ? 2 : (n <= 128 ? 4 : 8);
    const int G = (n + WR - 1) / WR, np = G * WR;
    // 32 columns of a state per CTA; 16 where the narrower tiles still find an SM each (every CTA is one chain of dependent
    // token steps: more, narrower CTAs shorten the step's critical path as long as they all run at once; measured at 2 x 1,024
    // tokens: 12 heads of 64: 209 -> 178 us; 32 heads of 64, whose 256 narrow CTAs exceed the SMs: 220 -> 240 us)
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        MLLM_CUDA(cudaGetDevice(&dev));
        MLLM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    if (want_cols != 0 && want_cols != 16 && want_cols != 32) return mllm_fail(1, "wkv_scan: %d columns per CTA (16, 32, or 0 for the rule)", want_cols);
    const int cols = want_cols ? want_cols : ((n > 16 && (long long)S * Hr * ((n + 15) / 16) <= sms) ? 16 : 32);
    const size_t smem = sizeof(float) * ((size_t)3 * WKV_CH * np + WKV_CH * cols + (size_t)G * WKV_CH * cols);
    if (smem > 200 * 1024) return mllm_fail(1, "wkv_scan: heads of %d need %zu bytes of shared memory", n, smem);
    WkvArgs a{cu_q, slots, u, state, state_stride, prev_off, r_stride, k_stride, v_stride, w_stride, o_stride, h_stride,
              Hr, n, D, write_state};
    const dim3 grid(S, Hr, (n + cols - 1) / cols), block(cols, G);
#define MLLM_WKV_C(TT, WRR, CC)                                                                                          \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            MLLM_CUDA(cudaFuncSetAttribute(wkv_scan_kernel<TT, WRR, CC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MLLM_CUDA(mllm_launch(wkv_scan_kernel<TT, WRR, CC>, grid, block, smem, stream, true, (const TT*)r, (const TT*)k, \
                              (const TT*)v, w, (const TT*)h, o, a));                                                     \
    } while (0)
#define MLLM_WKV(TT, WRR)                                                                                                \
    do {                                                                                                                 \
        if (cols == 16) MLLM_WKV_C(TT, WRR, 16); else MLLM_WKV_C(TT, WRR, 32);                                           \
    } while (0)
    if (dtype == MLLM_F32) {
        if (WR == 2) MLLM_WKV(float, 2); else if (WR == 4) MLLM_WKV(float, 4); else MLLM_WKV(float, 8);
    } else if (dtype == MLLM_BF16) {
        if (WR == 2) MLLM_WKV(__nv_bfloat16, 2); else if (WR == 4) MLLM_WKV(__nv_bfloat16, 4); else MLLM_WKV(__nv_bfloat16, 8);
    } else {
        return mllm_fail(1, "wkv_scan: unknown dtype code %d", dtype);
    }
#undef MLLM_WKV
#undef MLLM_WKV_C
    return 0;
}

MLLM_EXPORT int mllm_wkv_finish(const float* o, long long o_stride, const void* z, long long z_stride, const float* weight,
                                void* y, long long y_stride, int T, int Hr, int n, float eps, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long blocks = ((long long)T * Hr + 3) / 4;
    if (blocks > 2147483647LL) return mllm_fail(1, "wkv_finish: too many (token, head) pairs");
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(wkv_finish_kernel<float>, dim3((unsigned)blocks), dim3(128), 0, stream, true, o, o_stride,
                              (const float*)z, z_stride, weight, (float*)y, y_stride, T, Hr, n, eps));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(wkv_finish_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(128), 0, stream, true, o, o_stride,
                              (const __nv_bfloat16*)z, z_stride, weight, (__nv_bfloat16*)y, y_stride, T, Hr, n, eps));
    else
        return mllm_fail(1, "wkv_finish: unknown dtype code %d", dtype);
    return 0;
}

// 1 when the single-launch kernel for steps of single tokens takes heads of n entries with a decay of rank R
MLLM_EXPORT int mllm_wkv_step_ok(int n, int R) {
    if (n <= 0 || n > 128 || R <= 0) return 0;
    const int evp = (n + 31) / 32 * 32, G = 1024 / evp;
    const size_t smem = sizeof(float) * ((size_t)n * (R + 1) + R + 3 * (size_t)n + evp + (size_t)G * evp);
    return smem <= 160 * 1024 ? 1 : 0;
}

// The recurrence of a step of single tokens in one launch: decays from low [T, R], W2 and w0, the update of the state,
// o, and y = o / sqrt(mean(o^2) + eps) * weight * silu(z) per head, [T, Hr*n] in `dtype`.
MLLM_EXPORT int mllm_wkv_step(const void* r, long long r_stride, const void* k, long long k_stride, const void* v,
                              long long v_stride, const void* low, long long l_stride, const void* W2, const float* w0,
                              const float* u, const void* z, long long z_stride, const float* weight, const void* h,
                              long long h_stride, float* state, long long state_stride, long long prev_off, const int* cu_q,
                              const int* slots, void* y, long long y_stride, int S, int Hr, int n, int R, int D, float eps,
                              int write_state, int dtype, cudaStream_t stream) {
    if (S <= 0) return 0;
    if (!mllm_wkv_step_ok(n, R) || Hr <= 0 || Hr > 65535) return mllm_fail(1, "wkv_step: %d heads of %d, rank %d", Hr, n, R);
    const int evp = (n + 31) / 32 * 32, G = 1024 / evp;
    const int rk = (n + G - 1) / G;
    const size_t smem = sizeof(float) * ((size_t)n * (R + 1) + R + 3 * (size_t)n + evp + (size_t)G * evp);
    WkvArgs a{cu_q, slots, u, state, state_stride, prev_off, r_stride, k_stride, v_stride, 0, 0, h_stride, Hr, n, D, write_state};
    const dim3 grid(S, Hr), block(evp * G);
#define MLLM_STEP(TT, RKK)                                                                                               \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            MLLM_CUDA(cudaFuncSetAttribute(wkv_step_kernel<TT, RKK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MLLM_CUDA(mllm_launch(wkv_step_kernel<TT, RKK>, grid, block, smem, stream, true, (const TT*)r, (const TT*)k,    \
                              (const TT*)v, (const TT*)low, (const TT*)W2, w0, (const TT*)z, weight, (const TT*)h, (TT*)y, \
                              l_stride, z_stride, y_stride, R, evp, eps, a));                                            \
    } while (0)
    if (dtype == MLLM_F32) {
        if (rk <= 4) MLLM_STEP(float, 4); else MLLM_STEP(float, 16);
    } else if (dtype == MLLM_BF16) {
        if (rk <= 4) MLLM_STEP(__nv_bfloat16, 4); else MLLM_STEP(__nv_bfloat16, 16);
    } else {
        return mllm_fail(1, "wkv_step: unknown dtype code %d", dtype);
    }
#undef MLLM_STEP
    return 0;
}

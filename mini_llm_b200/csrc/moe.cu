// A routed feed-forward (mixture of experts) in which the host reads nothing back:
//
//   moe_route       a warp per token: router logits in 32-bit, softmax over all experts, the best `keep` of `n_groups`
//                   equal groups of neighbouring experts (a group's score is its largest), the `top` best experts inside
//                   those groups (the lowest index wins among equals), weights = scores / (their sum + 1e-20).
//                   With `bias` a number per expert is added to the logits first.  `mode` 1: no softmax over all
//                   experts: the `top` largest logits are chosen and the weights are the softmax over those alone.
//                   `mode` 2: the scores are sigmoid(logit), each expert's on its own.  `group_sum` 2: a group's score is
//                   the sum of its two largest scores instead of its largest.  The weights are multiplied by `w_scale`.
//   moe_sort        one CTA: the (token, choice) pairs ordered by expert (a counting sort) and the experts' offsets;
//                   with up to 16 tokens (decode steps) routing and ordering are one launch of one CTA.
//   moe_grouped     out[row] = A[a_row] W_e^T for the pairs of expert e; a CTA finds its expert from the offsets on the
//                   device, so the grid depends on the number of pairs only.  `gated`: W_e is [2F, K] (gate rows, then
//                   up rows) and the result is act(gate) * up (silu, or the clamped form of gate_mul); an expert without a
//                   gate has W_e [F, K] and an activation of one argument on the product (`uact`: the square of relu).  Three kernels: CUDA cores, 32 pairs x 64 columns per
//                   CTA (32-bit weights, odd sizes); tensor cores, 64 x 64 (bfloat16); and for up to 32 pairs (decode
//                   steps) a CTA per pair and 64 columns whose warps stream the weight rows.
//   moe_combine     y[t] (+)= sum_k weight[t][k] * pair_out[t * top + k], in the order of k.
// A row of a product depends on that row's input only, so a token's result does not depend on what else is in the batch.
#include "common.cuh"

namespace {

constexpr int MAX_E = 512;
constexpr int MOE_FEW_TOKENS = 16;    // up to this many tokens one CTA routes them all and orders the pairs in the same launch
constexpr int MOE_FEW_PAIRS = 32;     // up to this many (token, choice) pairs every pair streams its expert's weights itself

// One warp routes one token; `s` is the warp's E floats of shared memory.
template <typename T>
__device__ __forceinline__ void route_token(const T* x, const T* __restrict__ Wr, const float* __restrict__ bias, int mode,
                                            float* s, int D, int E, int top, int n_groups, int keep, int group_sum,
                                            float w_scale, int* idx, float* wout, int lane) {
    constexpr int V = 16 / sizeof(T);                           // elements per 16-byte load
    const bool vec = D % V == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)Wr % 16 == 0;
    for (int e0 = 0; e0 < E; e0 += 4) {                         // four experts at a time: their loads are in flight together
        float a[4] = {0.f, 0.f, 0.f, 0.f};
        const T* w0 = Wr + (size_t)e0 * D;
        const T* w1 = Wr + (size_t)min(e0 + 1, E - 1) * D;
        const T* w2 = Wr + (size_t)min(e0 + 2, E - 1) * D;
        const T* w3 = Wr + (size_t)min(e0 + 3, E - 1) * D;
        if (vec) {
#pragma unroll 2
            for (int d = lane * V; d < D; d += 32 * V) {
                const uint4 xv = *reinterpret_cast<const uint4*>(x + d);
                const uint4 v0 = *reinterpret_cast<const uint4*>(w0 + d), v1 = *reinterpret_cast<const uint4*>(w1 + d);
                const uint4 v2 = *reinterpret_cast<const uint4*>(w2 + d), v3 = *reinterpret_cast<const uint4*>(w3 + d);
                const T* px = reinterpret_cast<const T*>(&xv);
                const T* p0 = reinterpret_cast<const T*>(&v0);
                const T* p1 = reinterpret_cast<const T*>(&v1);
                const T* p2 = reinterpret_cast<const T*>(&v2);
                const T* p3 = reinterpret_cast<const T*>(&v3);
#pragma unroll
                for (int c = 0; c < V; ++c) {
                    const float xf = to_f32(px[c]);
                    a[0] = fmaf(xf, to_f32(p0[c]), a[0]);
                    a[1] = fmaf(xf, to_f32(p1[c]), a[1]);
                    a[2] = fmaf(xf, to_f32(p2[c]), a[2]);
                    a[3] = fmaf(xf, to_f32(p3[c]), a[3]);
                }
            }
        } else {
#pragma unroll 4
            for (int d = lane; d < D; d += 32) {
                const float xv = to_f32(x[d]);
                a[0] = fmaf(xv, to_f32(w0[d]), a[0]);
                a[1] = fmaf(xv, to_f32(w1[d]), a[1]);
                a[2] = fmaf(xv, to_f32(w2[d]), a[2]);
                a[3] = fmaf(xv, to_f32(w3[d]), a[3]);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const float v = warp_sum(a[u]);
            if (lane == 0 && e0 + u < E) s[e0 + u] = v + (bias ? bias[e0 + u] : 0.f);
        }
    }
    __syncwarp();
    if (mode == 1) {
        // the largest logits, and a softmax over them alone
        if (lane == 0) {
            float mx = -INFINITY, wsum = 0.f;
            for (int k = 0; k < top; ++k) {
                int best = 0;
                float bv = -INFINITY;
                for (int e = 0; e < E; ++e)
                    if (s[e] > bv) { bv = s[e]; best = e; }
                if (k == 0) mx = bv;
                idx[k] = best;
                wout[k] = expf(bv - mx);
                wsum += wout[k];
                s[best] = -INFINITY;                             // taken
            }
            for (int k = 0; k < top; ++k) wout[k] = wout[k] / wsum * w_scale;
        }
        __syncwarp();
        return;
    }
    if (mode == 2) {
        for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-s[e]));
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < E; e += 32) mx = fmaxf(mx, s[e]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) {
            const float v = expf(s[e] - mx);
            s[e] = v;
            sum += v;
        }
        sum = warp_sum(sum);
        __syncwarp();
        for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
    }
    __syncwarp();
    if (lane == 0) {
        // experts outside the kept groups are marked by a negative score (scores are >= 0)
        if (n_groups > 1 && keep < n_groups) {
            const int per = E / n_groups;
            unsigned long long kept = 0ull;                 // at most 64 groups
            for (int k = 0; k < keep; ++k) {
                int best = -1;
                float bv = -1.f;
                for (int g = 0; g < n_groups; ++g) {
                    if ((kept >> g) & 1ull) continue;
                    float gm = -1.f, g2 = 0.f;             // the largest score of the group and the one after it
                    for (int e = g * per; e < (g + 1) * per; ++e) {
                        if (s[e] > gm) { g2 = fmaxf(gm, 0.f); gm = s[e]; }
                        else if (s[e] > g2) g2 = s[e];
                    }
                    if (group_sum == 2 && per > 1) gm += g2;
                    if (gm > bv) { bv = gm; best = g; }
                }
                if (best >= 0) kept |= 1ull << best;
            }
            for (int g = 0; g < n_groups; ++g)
                if (!((kept >> g) & 1ull))
                    for (int e = g * per; e < (g + 1) * per; ++e) s[e] = -1.f - s[e];
        }
        float wsum = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float bv = -INFINITY;
            for (int e = 0; e < E; ++e)
                if (s[e] > bv) { bv = s[e]; best = e; }
            idx[k] = best;
            wout[k] = bv;
            wsum += bv;
            s[best] = -8.f;                                  // taken
        }
        for (int k = 0; k < top; ++k) wout[k] = wout[k] / (wsum + 1e-20f) * w_scale;
    }
    __syncwarp();
}

// The (token, choice) pairs ordered by expert: offsets[E + 1], sorted[n] = pair ids (pairs of one expert in pair order).
// All threads of the CTA; cnt holds E + 1 ints of shared memory.
__device__ __forceinline__ void sort_pairs(const int* idx, int n, int E, int* offsets, int* sorted, int* cnt) {
    for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) atomicAdd(&cnt[idx[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            const int c = cnt[e];
            cnt[e] = run;
            run += c;
        }
        cnt[E] = run;
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = cnt[e];
    // a warp per expert walks the pairs in order: a stable order without atomics
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int e = warp; e < E; e += nw) {
        int at = cnt[e];
        for (int i0 = 0; i0 < n; i0 += 32) {
            const int i = i0 + lane;
            const bool mine = i < n && idx[i] == e;
            const unsigned ballot = __ballot_sync(0xffffffffu, mine);
            if (mine) sorted[at + __popc(ballot & ((1u << lane) - 1u))] = i;
            at += __popc(ballot);
        }
    }
}

// 4 warps, a token each; dynamic shared memory: 4 * E floats
template <typename T>
__global__ void __launch_bounds__(128)
moe_route_kernel(const T* h, long long ld, const T* __restrict__ Wr, const float* __restrict__ bias, int mode, int Tn, int D,
                 int E, int top, int n_groups, int keep, int group_sum, float w_scale, int* idx, float* wout) {
    extern __shared__ float sc[];
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= Tn) return;
    route_token(h + (size_t)t * ld, Wr, bias, mode, sc + warp * E, D, E, top, n_groups, keep, group_sum, w_scale,
                idx + (size_t)t * top, wout + (size_t)t * top, lane);
}

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* idx, int n, int E, int* offsets, int* sorted) {
    __shared__ int cnt[MAX_E + 1];
    pdl_wait();
    sort_pairs(idx, n, E, offsets, sorted, cnt);
}

// Few tokens (decode steps): one CTA of 8 warps routes them all and orders the pairs, in one launch.
// dynamic shared memory: 8 * E floats, then E + 1 ints
template <typename T>
__global__ void __launch_bounds__(256)
moe_route_sort_kernel(const T* h, long long ld, const T* __restrict__ Wr, const float* __restrict__ bias, int mode, int Tn,
                      int D, int E, int top, int n_groups, int keep, int group_sum, float w_scale, int* idx, float* wout,
                      int* offsets, int* sorted) {
    extern __shared__ float sc[];
    int* cnt = reinterpret_cast<int*>(sc + 8 * E);
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int t = warp; t < Tn; t += 8)
        route_token(h + (size_t)t * ld, Wr, bias, mode, sc + warp * E, D, E, top, n_groups, keep, group_sum, w_scale,
                    idx + (size_t)t * top, wout + (size_t)t * top, lane);
    __syncthreads();                                         // the CTA's own writes of idx are visible to all its threads
    sort_pairs(idx, Tn * top, E, offsets, sorted, cnt);
}

// an activation of one argument on a product (an expert without a gate); 0: none
__device__ __forceinline__ float unary_act(float v, int uact) {
    if (uact == MLLM_ACT_RELU_SQ) { const float r = fmaxf(v, 0.f); return r * r; }
    if (uact == MLLM_ACT_RELU) return fmaxf(v, 0.f);
    if (uact == MLLM_ACT_GELU_TANH) return gelu_tanh_f(v);
    return v;
}

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const TA* A, long long lda, const TW* __restrict__ W, TO* out, long long ldo, const int* offsets,
                   const int* sorted, int E, int N, int K, int a_div, int out_by_pair, int gated, float limit, float alpha,
                   int uact) {
    __shared__ float As[32][33];
    __shared__ float Ws[64][33];
    __shared__ float Us[64][33];
    __shared__ int rows_a[32], rows_o[32];
    __shared__ int s_e, s_r0, s_cnt;
    pdl_wait();
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, e = 0, found = -1, r0 = 0, c = 0;
        for (; e < E; ++e) {
            const int lo = offsets[e], n = offsets[e + 1] - lo;
            const int tiles = (n + 31) / 32;
            if (tile < tiles) { found = e; r0 = lo + tile * 32; c = min(32, n - tile * 32); break; }
            tile -= tiles;
        }
        s_e = found; s_r0 = r0; s_cnt = c;
    }
    __syncthreads();
    const int e = s_e, cnt = s_cnt;
    if (e < 0) return;
    if (threadIdx.x < 32) {
        const int i = s_r0 + threadIdx.x;
        const int pair = threadIdx.x < cnt ? sorted[i] : 0;
        rows_a[threadIdx.x] = a_div > 0 ? pair / a_div : i;
        rows_o[threadIdx.x] = out_by_pair ? pair : i;
    }
    __syncthreads();
    const int n0 = blockIdx.y * 64;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    const size_t wrows = gated ? (size_t)2 * N : (size_t)N;
    const TW* We = W + (size_t)e * wrows * K;
    float acc[2][4] = {}, acu[2][4] = {};
    for (int k0 = 0; k0 < K; k0 += 32) {
        for (int i = threadIdx.x; i < 32 * 32; i += 256) {
            const int r = i >> 5, c = i & 31;
            As[r][c] = (r < cnt && k0 + c < K) ? to_f32(A[(size_t)rows_a[r] * lda + k0 + c]) : 0.f;
        }
        for (int i = threadIdx.x; i < 64 * 32; i += 256) {
            const int r = i >> 5, c = i & 31;
            const bool ok = n0 + r < N && k0 + c < K;
            Ws[r][c] = ok ? to_f32(We[(size_t)(n0 + r) * K + k0 + c]) : 0.f;
            if (gated) Us[r][c] = ok ? to_f32(We[(size_t)(N + n0 + r) * K + k0 + c]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < 32; ++kk) {
            const float a0 = As[ty * 2][kk], a1 = As[ty * 2 + 1][kk];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float w = Ws[tx + 16 * i][kk];
                acc[0][i] = fmaf(a0, w, acc[0][i]);
                acc[1][i] = fmaf(a1, w, acc[1][i]);
            }
            if (gated) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float u = Us[tx + 16 * i][kk];
                    acu[0][i] = fmaf(a0, u, acu[0][i]);
                    acu[1][i] = fmaf(a1, u, acu[1][i]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int r = ty * 2 + j;
        if (r >= cnt) continue;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int n = n0 + tx + 16 * i;
            if (n >= N) continue;
            float v = acc[j][i];
            if (gated) v = gate_mul(v, acu[j][i], gated, limit, alpha);
            else v = unary_act(v, uact);
            out[(size_t)rows_o[r] * ldo + n] = from_f32<TO>(v);
        }
    }
}

// ------------------------------------------------------------------------------------------------ few pairs (decode steps)
// grid (pairs, column blocks of 64), 8 warps.  The pair's input row is staged in shared memory as 32-bit; a warp owns 8
// columns, its lanes split K with 16-byte loads of the 8 weight rows (all in flight at once), and the sums meet by
// a butterfly.  Every weight of the pair's expert leaves L2 once per pair: with few pairs that is the whole cost.
template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const TA* A, long long lda, const TW* __restrict__ W, TO* out, long long ldo, const int* offsets,
                const int* sorted, int E, int N, int K, int a_div, int out_by_pair, int gated, float limit, float alpha,
                int uact) {
    extern __shared__ float xs[];                                // [K]
    __shared__ int s_e;
    pdl_wait();
    const int i = blockIdx.x;
    if (threadIdx.x == 0) {
        int e = 0;
        while (e < E - 1 && offsets[e + 1] <= i) ++e;
        s_e = e;
    }
    const int pair = sorted[i];
    const TA* a = A + (size_t)(a_div > 0 ? pair / a_div : i) * lda;
    for (int k = threadIdx.x; k < K; k += 256) xs[k] = to_f32(a[k]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * 64 + warp * 8;
    if (n0 >= N) return;
    const size_t wrows = gated ? (size_t)2 * N : (size_t)N;
    const TW* We = W + (size_t)s_e * wrows * K;
    constexpr int V = 16 / sizeof(TW);                           // weights per 16-byte load
    float acc[8], acu[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = acu[u] = 0.f;
    const bool vec = K % V == 0 && ((uintptr_t)W % 16 == 0);
    if (vec) {
        for (int k = lane * V; k < K; k += 32 * V) {
            uint4 w[8], wu[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int n = min(n0 + u, N - 1);
                w[u] = *reinterpret_cast<const uint4*>(We + (size_t)n * K + k);
                if (gated) wu[u] = *reinterpret_cast<const uint4*>(We + (size_t)(N + n) * K + k);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const TW* p = reinterpret_cast<const TW*>(&w[u]);
                const TW* q = reinterpret_cast<const TW*>(&wu[u]);
#pragma unroll
                for (int c = 0; c < V; ++c) {
                    acc[u] = fmaf(xs[k + c], to_f32(p[c]), acc[u]);
                    if (gated) acu[u] = fmaf(xs[k + c], to_f32(q[c]), acu[u]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int n = min(n0 + u, N - 1);
                acc[u] = fmaf(xs[k], to_f32(We[(size_t)n * K + k]), acc[u]);
                if (gated) acu[u] = fmaf(xs[k], to_f32(We[(size_t)(N + n) * K + k]), acu[u]);
            }
        }
    }
    const size_t orow = (size_t)(out_by_pair ? pair : i) * ldo;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
        float v = warp_sum(acc[u]);
        if (gated) v = gate_mul(v, warp_sum(acu[u]), gated, limit, alpha);
        else v = unary_act(v, uact);
        if (lane == 0 && n0 + u < N) out[orow + n0 + u] = from_f32<TO>(v);
    }
}

// ------------------------------------------------------------------------------------------------ many pairs, bfloat16
// The same products on tensor cores (mma.sync m16n8k16, 32-bit accumulators): 64 pairs x 64 columns per CTA (with
// `gated` 64 gate and 64 up columns), K in steps of 64 staged by cp.async (input rows gathered by pair), the next step's
// while the current one is multiplied.  A warp owns 16 pairs.
constexpr int GM = 64, GN = 64, GK = 64, GROW = GK + 8;

__device__ __forceinline__ void g_ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void g_ldsm_x2(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void g_mma(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void g_cp16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

template <typename TO, int GATED>
__global__ void __launch_bounds__(128)
moe_grouped_mma_kernel(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* __restrict__ W, TO* out, long long ldo,
                       const int* offsets, const int* sorted, int E, int N, int K, int a_div, int out_by_pair, int act,
                       float limit, float alpha) {
    using bf = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char gsm[];
    constexpr int STAGE = (GM + GN * (1 + GATED)) * GROW;        // elements per stage
    bf* sm = reinterpret_cast<bf*>(gsm);
    __shared__ int rows_a[GM], rows_o[GM];
    __shared__ int s_e, s_r0, s_cnt;
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        int tile = blockIdx.x, found = -1, r0 = 0, c = 0;
        for (int e = 0; e < E; ++e) {
            const int lo = offsets[e], n = offsets[e + 1] - lo;
            const int tiles = (n + GM - 1) / GM;
            if (tile < tiles) { found = e; r0 = lo + tile * GM; c = min(GM, n - tile * GM); break; }
            tile -= tiles;
        }
        s_e = found; s_r0 = r0; s_cnt = c;
    }
    __syncthreads();
    const int e = s_e, cnt = s_cnt;
    if (e < 0) return;
    if (tid < GM) {
        const int i = s_r0 + tid;
        const int pair = tid < cnt ? sorted[i] : 0;
        rows_a[tid] = a_div > 0 ? pair / a_div : (tid < cnt ? i : s_r0);
        rows_o[tid] = out_by_pair ? pair : i;
    }
    __syncthreads();
    const int n0 = blockIdx.y * GN;
    const bf* We = W + (size_t)e * (size_t)(1 + GATED) * N * K;
    auto stage = [&](int k0, int buf) {
        bf* As = sm + buf * STAGE;
        bf* Ws = As + GM * GROW;
        for (int i = tid; i < GM * 8; i += 128) {
            const int r = i >> 3, pc = i & 7, k = k0 + pc * 8;
            const bool ok = r < cnt && k < K;
            g_cp16(As + r * GROW + pc * 8, ok ? A + (size_t)rows_a[r] * lda + k : A, ok);
        }
        for (int i = tid; i < GN * 8 * (1 + GATED); i += 128) {
            const int r = i >> 3, pc = i & 7, k = k0 + pc * 8;
            const int n = r < GN ? n0 + r : N + n0 + (r - GN);     // gate rows, then up rows
            const bool ok = (r < GN ? n0 + r : n0 + r - GN) < N && k < K;
            g_cp16(Ws + r * GROW + pc * 8, ok ? We + (size_t)n * K + k : We, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    float acc[8][4], acu[GATED ? 8 : 1][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f; }
#pragma unroll
    for (int n = 0; n < (GATED ? 8 : 1); ++n) { acu[n][0] = acu[n][1] = acu[n][2] = acu[n][3] = 0.f; }
    const int nk = (K + GK - 1) / GK;
    stage(0, 0);
    for (int t = 0; t < nk; ++t) {
        const int buf = t & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        if (t + 1 < nk) stage((t + 1) * GK, buf ^ 1);
        const bf* As = sm + buf * STAGE;
        const bf* Ws = As + GM * GROW;
#pragma unroll
        for (int kk = 0; kk < GK; kk += 16) {
            uint32_t af[4];
            g_ldsm_x4(af, As + (warp * 16 + (lane & 15)) * GROW + kk + (lane >> 4) * 8);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                uint32_t b[2];
                g_ldsm_x2(b, Ws + (n * 8 + (lane & 7)) * GROW + kk + ((lane >> 3) & 1) * 8);
                g_mma(acc[n], af, b);
                if (GATED) {
                    g_ldsm_x2(b, Ws + (GN + n * 8 + (lane & 7)) * GROW + kk + ((lane >> 3) & 1) * 8);
                    g_mma(acu[n], af, b);
                }
            }
        }
    }
    const int r0 = warp * 16 + (lane >> 2);
#pragma unroll
    for (int n = 0; n < 8; ++n) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int r = r0 + (c >> 1) * 8, col = n0 + n * 8 + 2 * (lane & 3) + (c & 1);
            if (r < cnt && col < N) {
                float v = acc[n][c];
                if (GATED) v = gate_mul(v, acu[n][c], act, limit, alpha);
                else v = unary_act(v, act);
                out[(size_t)rows_o[r] * ldo + col] = from_f32<TO>(v);
            }
        }
    }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* pair_out, const float* w, float* y, long long ldy, int Tn, int D, int top, int accumulate) {
    pdl_wait();
    const long long total = (long long)Tn * D;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / D), d = (int)(i % D);
        float a = accumulate ? y[(size_t)t * ldy + d] : 0.f;
        for (int k = 0; k < top; ++k) a = fmaf(w[(size_t)t * top + k], pair_out[((size_t)t * top + k) * D + d], a);
        y[(size_t)t * ldy + d] = a;
    }
}

}  // namespace

MLLM_EXPORT int mllm_moe_max_experts() { return MAX_E; }

MLLM_EXPORT int mllm_moe_route(const void* h, long long ld, const void* Wr, const float* bias, int mode, int Tn, int D, int E,
                               int top, int n_groups, int keep, int group_sum, float w_scale, int* idx, float* w, int* offsets,
                               int* sorted, int dtype, cudaStream_t stream) {
    if (Tn <= 0) return 0;
    if (mode < 0 || mode > 2) return mllm_fail(1, "moe_route: unknown mode %d", mode);
    if (group_sum != 1 && group_sum != 2) return mllm_fail(1, "moe_route: a group's score is its largest score or the sum of its two largest, not of %d", group_sum);
    if (mode == 1 && n_groups != 1) return mllm_fail(1, "moe_route: the softmax over the chosen logits takes no groups");
    if (E < 1 || E > MAX_E || top < 1 || top > E) return mllm_fail(1, "moe_route: %d experts (at most %d), top %d", E, MAX_E, top);
    if (n_groups < 1 || E % n_groups || keep < 1 || keep > n_groups || n_groups > 64)
        return mllm_fail(1, "moe_route: %d experts in %d groups (at most 64), %d kept", E, n_groups, keep);
    if (keep * (E / n_groups) < top) return mllm_fail(1, "moe_route: %d kept groups of %d experts cannot give %d", keep, E / n_groups, top);
    if (Tn <= MOE_FEW_TOKENS) {
        const size_t smem = (size_t)8 * E * 4 + (size_t)(E + 1) * 4;
        if (dtype == MLLM_F32)
            MLLM_CUDA(mllm_launch(moe_route_sort_kernel<float>, dim3(1), dim3(256), smem, stream, true, (const float*)h, ld,
                                  (const float*)Wr, bias, mode, Tn, D, E, top, n_groups, keep, group_sum, w_scale, idx, w, offsets, sorted));
        else if (dtype == MLLM_BF16)
            MLLM_CUDA(mllm_launch(moe_route_sort_kernel<__nv_bfloat16>, dim3(1), dim3(256), smem, stream, true,
                                  (const __nv_bfloat16*)h, ld, (const __nv_bfloat16*)Wr, bias, mode, Tn, D, E, top, n_groups, keep,
                                  group_sum, w_scale, idx, w, offsets, sorted));
        else
            return mllm_fail(1, "moe_route: unknown dtype code %d", dtype);
        return 0;
    }
    const size_t smem = (size_t)4 * E * 4;
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(moe_route_kernel<float>, dim3((Tn + 3) / 4), dim3(128), smem, stream, true, (const float*)h, ld,
                              (const float*)Wr, bias, mode, Tn, D, E, top, n_groups, keep, group_sum, w_scale, idx, w));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(moe_route_kernel<__nv_bfloat16>, dim3((Tn + 3) / 4), dim3(128), smem, stream, true,
                              (const __nv_bfloat16*)h, ld, (const __nv_bfloat16*)Wr, bias, mode, Tn, D, E, top, n_groups, keep,
                              group_sum, w_scale, idx, w));
    else
        return mllm_fail(1, "moe_route: unknown dtype code %d", dtype);
    MLLM_CUDA(mllm_launch(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, true, (const int*)idx, Tn * top, E, offsets, sorted));
    return 0;
}

MLLM_EXPORT int mllm_moe_few_tokens() { return MOE_FEW_TOKENS; }

// kind 0: A in `dtype`, gated, out in `dtype` (the experts' first product with its activation `act`: MLLM_ACT_SILU, or
// MLLM_ACT_SWIGLU_CLAMP with `limit` and `alpha`);
// kind 1: A in `dtype`, out 32-bit (the experts' second product);
// kind 2: A in `dtype`, no gate, out in `dtype` = act(A W_e^T) with an activation of one argument (MLLM_ACT_RELU_SQ ...):
// the first product of experts without a gate.
MLLM_EXPORT int mllm_moe_grouped(const void* A, long long lda, const void* W, void* out, long long ldo, const int* offsets,
                                 const int* sorted, int n_pairs, int E, int N, int K, int a_div, int out_by_pair, int kind,
                                 int act, float limit, float alpha, int dtype, cudaStream_t stream) {
    if (n_pairs <= 0 || N <= 0) return 0;
    const dim3 grid((n_pairs + 31) / 32 + E, (N + 63) / 64), block(256);
    if (grid.y > 65535) return mllm_fail(1, "moe_grouped: too many columns");
    if (kind == 0 && act != MLLM_ACT_SILU && act != MLLM_ACT_SWIGLU_CLAMP) return mllm_fail(1, "moe_grouped: activation code %d", act);
    if (kind == 2 && act != MLLM_ACT_RELU_SQ && act != MLLM_ACT_RELU && act != MLLM_ACT_GELU_TANH)
        return mllm_fail(1, "moe_grouped: activation code %d of an expert without a gate", act);
    if (kind < 0 || kind > 2) return mllm_fail(1, "moe_grouped: kind %d", kind);
    const int gated = kind == 0 ? act : 0;
    const int uact = kind == 2 ? act : 0;
    if (n_pairs <= MOE_FEW_PAIRS && (size_t)K * 4 <= 96 * 1024) {
        const dim3 fg(n_pairs, (N + 63) / 64);
        const size_t smem = (size_t)K * 4;
#define MLLM_ROWS(TA, TW, TO)                                                                                            \
        do {                                                                                                             \
            static bool raised = false;                                                                                  \
            if (smem > 48 * 1024 && !raised) {                                                                           \
                MLLM_CUDA(cudaFuncSetAttribute(moe_rows_kernel<TA, TW, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024)); \
                raised = true;                                                                                           \
            }                                                                                                            \
            MLLM_CUDA(mllm_launch(moe_rows_kernel<TA, TW, TO>, fg, block, smem, stream, true, (const TA*)A, lda, (const TW*)W, \
                                  (TO*)out, ldo, offsets, sorted, E, N, K, a_div, out_by_pair, gated, limit, alpha, uact)); \
        } while (0)
        if (dtype == MLLM_F32) MLLM_ROWS(float, float, float);
        else if (dtype == MLLM_BF16 && kind != 1) MLLM_ROWS(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
        else if (dtype == MLLM_BF16) MLLM_ROWS(__nv_bfloat16, __nv_bfloat16, float);
        else return mllm_fail(1, "moe_grouped: unknown dtype code %d", dtype);
#undef MLLM_ROWS
        return 0;
    }
    if (dtype == MLLM_BF16 && K % 8 == 0 && lda % 8 == 0 && (uintptr_t)A % 16 == 0 && (uintptr_t)W % 16 == 0) {
        const dim3 mg((n_pairs + GM - 1) / GM + E, (N + GN - 1) / GN);
        if (kind == 0) {
            constexpr size_t smem = (size_t)2 * (GM + 2 * GN) * GROW * 2;
            static bool raised = false;
            if (!raised) {
                MLLM_CUDA(cudaFuncSetAttribute(moe_grouped_mma_kernel<__nv_bfloat16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
                raised = true;
            }
            MLLM_CUDA(mllm_launch(moe_grouped_mma_kernel<__nv_bfloat16, 1>, mg, dim3(128), smem, stream, true, (const __nv_bfloat16*)A,
                                  lda, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, ldo, offsets, sorted, E, N, K, a_div, out_by_pair, act, limit,
                                  alpha));
        } else if (kind == 2) {
            constexpr size_t smem = (size_t)2 * (GM + GN) * GROW * 2;
            MLLM_CUDA(mllm_launch(moe_grouped_mma_kernel<__nv_bfloat16, 0>, mg, dim3(128), smem, stream, true, (const __nv_bfloat16*)A, lda,
                                  (const __nv_bfloat16*)W, (__nv_bfloat16*)out, ldo, offsets, sorted, E, N, K, a_div, out_by_pair, act, 0.f, 0.f));
        } else {
            constexpr size_t smem = (size_t)2 * (GM + GN) * GROW * 2;
            MLLM_CUDA(mllm_launch(moe_grouped_mma_kernel<float, 0>, mg, dim3(128), smem, stream, true, (const __nv_bfloat16*)A, lda,
                                  (const __nv_bfloat16*)W, (float*)out, ldo, offsets, sorted, E, N, K, a_div, out_by_pair, 0, 0.f, 0.f));
        }
        return 0;
    }
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(moe_grouped_kernel<float, float, float>, grid, block, 0, stream, true, (const float*)A, lda,
                              (const float*)W, (float*)out, ldo, offsets, sorted, E, N, K, a_div, out_by_pair, gated, limit, alpha, uact));
    else if (dtype == MLLM_BF16 && kind != 1)
        MLLM_CUDA(mllm_launch(moe_grouped_kernel<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream, true,
                              (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, ldo, offsets, sorted, E,
                              N, K, a_div, out_by_pair, gated, limit, alpha, uact));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(moe_grouped_kernel<__nv_bfloat16, __nv_bfloat16, float>, grid, block, 0, stream, true,
                              (const __nv_bfloat16*)A, lda, (const __nv_bfloat16*)W, (float*)out, ldo, offsets, sorted, E, N, K,
                              a_div, out_by_pair, gated, limit, alpha, uact));
    else
        return mllm_fail(1, "moe_grouped: unknown dtype code %d", dtype);
    return 0;
}

MLLM_EXPORT int mllm_moe_combine(const float* pair_out, const float* w, float* y, long long ldy, int Tn, int D, int top,
                                 int accumulate, cudaStream_t stream) {
    if (Tn <= 0) return 0;
    const long long total = (long long)Tn * D;
    const int grid = (int)((total + 255) / 256 < 16384 ? (total + 255) / 256 : 16384);
    MLLM_CUDA(mllm_launch(moe_combine_kernel, dim3(grid), dim3(256), 0, stream, true, pair_out, w, y, ldy, Tn, D, top,
                          accumulate));
    return 0;
}

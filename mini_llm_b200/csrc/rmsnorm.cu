// RMS norm of 32-bit rows: y = x / sqrt(mean(x^2) + eps) * (w + offset), optionally of gathered rows,
// written as 32-bit or bfloat16.  `offset` is 1 for weights that are stored around zero and 0 for plain
// weights.  A second weight vector and output may be given: two norms of the same rows that differ only
// in their weights (the two branches of a parallel block) then cost one read of x and one sum of squares.
// With `heads` > 1 a row of x and of the output holds that many vectors of width D side by side, each normed on its
// own with the same weights (the per-head norm of a mixer's outputs); `scale` multiplies the result.
// All arithmetic is 32-bit; the sum of squares runs in an order that depends on the width only.
#include "common.cuh"

namespace {

template <typename TOut>
__global__ void rmsnorm_kernel(const float* x, long long x_stride, const int* __restrict__ rows,
                               const float* __restrict__ w1, const float* __restrict__ w2, TOut* __restrict__ out1,
                               TOut* __restrict__ out2, long long out_stride, int heads, int D, float eps, float offset,
                               float scale) {
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch();
    const int r = blockIdx.x / heads, hd = blockIdx.x % heads;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * x_stride + (size_t)hd * D;
    out1 += (size_t)r * out_stride + (size_t)hd * D;
    if (out2) out2 += (size_t)r * out_stride + (size_t)hd * D;
    float q = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) q = fmaf(xr[d], xr[d], q);
    const float inv = scale / sqrtf(block_sum(q, scratch) / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float y = xr[d] * inv;
        out1[d] = from_f32<TOut>(y * (w1[d] + offset));
        if (out2) out2[d] = from_f32<TOut>(y * (w2[d] + offset));
    }
}

template <typename TOut>
__device__ __forceinline__ void store4(TOut* o, float y0, float y1, float y2, float y3) {
    if constexpr (sizeof(TOut) == 4) {
        *reinterpret_cast<float4*>(o) = make_float4(y0, y1, y2, y3);
    } else {
        uint2 pk;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&pk);
        h[0] = __floats2bfloat162_rn(y0, y1);
        h[1] = __floats2bfloat162_rn(y2, y3);
        *reinterpret_cast<uint2*>(o) = pk;
    }
}

// One warp per row, the row held in registers (up to 2048 columns), 16-byte loads and stores.
template <typename TOut>
__global__ void __launch_bounds__(256)
rmsnorm_warp_kernel(const float* x, long long x_stride, const int* __restrict__ rows, const float* __restrict__ w1,
                    const float* __restrict__ w2, TOut* __restrict__ out1, TOut* __restrict__ out2, long long out_stride,
                    int heads, int R, int D, float eps, float offset, float scale) {
    constexpr int KEEP = 16;
    pdl_wait();
    pdl_launch();
    const int rh = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (rh >= R * heads) return;
    const int r = rh / heads, hd = rh % heads;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * x_stride + (size_t)hd * D;
    out1 += (size_t)r * out_stride + (size_t)hd * D;
    if (out2) out2 += (size_t)r * out_stride + (size_t)hd * D;
    float4 v[KEEP];
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int k = lane * 4 + i * 128;
        v[i] = k < D ? *reinterpret_cast<const float4*>(xr + k) : make_float4(0.f, 0.f, 0.f, 0.f);
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
    }
    const float inv = scale / sqrtf(warp_sum(q) / (float)D + eps);
#pragma unroll
    for (int i = 0; i < KEEP; ++i) {
        const int k = lane * 4 + i * 128;
        if (k >= D) break;
        const float y0 = v[i].x * inv, y1 = v[i].y * inv, y2 = v[i].z * inv, y3 = v[i].w * inv;
        const float4 g = __ldg(reinterpret_cast<const float4*>(w1 + k));
        store4<TOut>(out1 + k, y0 * (g.x + offset), y1 * (g.y + offset), y2 * (g.z + offset),
                     y3 * (g.w + offset));
        if (out2) {
            const float4 g2 = __ldg(reinterpret_cast<const float4*>(w2 + k));
            store4<TOut>(out2 + k, y0 * (g2.x + offset), y1 * (g2.y + offset), y2 * (g2.z + offset),
                         y3 * (g2.w + offset));
        }
    }
}

template <typename TOut>
int launch(const float* x, long long x_stride, const int* rows, const float* w1, const float* w2, void* out1, void* out2,
           long long out_stride, int heads, int R, int D, float eps, float offset, float scale, cudaStream_t stream) {
    constexpr int OV = 16 / sizeof(TOut);       // output elements per 16 bytes (stores are 16 or 8 bytes of 4 values)
    const bool fast = D % 4 == 0 && D <= 2048 && x_stride % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w1 % 16 == 0 &&
                      (uintptr_t)out1 % 16 == 0 && out_stride % OV == 0 && (heads == 1 || D % OV == 0) &&
                      (!out2 || ((uintptr_t)w2 % 16 == 0 && (uintptr_t)out2 % 16 == 0));
    if ((long long)R * heads > 2147483647LL) return mllm_fail(1, "rmsnorm: too many rows");
    if (fast) {
        MLLM_CUDA(mllm_launch(rmsnorm_warp_kernel<TOut>, dim3((R * heads + 7) / 8), dim3(256), 0, stream, true, x, x_stride,
                              rows, w1, w2, (TOut*)out1, (TOut*)out2, out_stride, heads, R, D, eps, offset, scale));
        return 0;
    }
    const int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : ((D + 31) / 32) * 32);
    MLLM_CUDA(mllm_launch(rmsnorm_kernel<TOut>, dim3(R * heads), dim3(threads), 0, stream, true, x, x_stride, rows, w1, w2,
                          (TOut*)out1, (TOut*)out2, out_stride, heads, D, eps, offset, scale));
    return 0;
}

// out[t][c] = act(gu[t][c]) * gu[t][F + c]: the gate and the up half of one product's output.
template <typename T>
__global__ void __launch_bounds__(256)
gated_act_kernel(const T* gu, long long gu_stride, T* __restrict__ out, long long out_stride, int rows, int F, int act,
                 float limit, float alpha) {
    pdl_wait();
    pdl_launch();
    const long long total = (long long)rows * F;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / F), c = (int)(i % F);
        const float g = to_f32(gu[(size_t)t * gu_stride + c]), u = to_f32(gu[(size_t)t * gu_stride + F + c]);
        out[(size_t)t * out_stride + c] = from_f32<T>(gate_mul(g, u, act, limit, alpha));
    }
}

// x[r] += (v / sqrt(mean(v^2) + eps) * w) * ls with v = y[r] (+ sum_k pw[r][k] * pairs[r * top + k], the weighted
// results of a routed feed-forward's chosen experts, in the order of k): a branch's result, normed, scaled per column and
// added to the 32-bit residual stream in one pass (ls, y or the pairs may be absent).  With `nw` the new x is normed once
// more, h = x / sqrt(mean(x^2) + neps) * (nw + noff), for the branch that reads it next.  The row is kept in shared memory.
template <typename TOut>
__global__ void __launch_bounds__(256)
join_kernel(const float* y, long long y_stride, const float* pairs, const float* pw, int top, const float* __restrict__ w,
            const float* __restrict__ ls, float* x, long long x_stride, const float* __restrict__ nw, float noff, float neps,
            TOut* h, long long h_stride, int D, float eps) {
    extern __shared__ float rowbuf[];       // [D]
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch();
    const size_t r = blockIdx.x;
    float* xr = x + r * x_stride;
    float q = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = y ? y[r * y_stride + d] : 0.f;
        if (pairs)
            for (int k = 0; k < top; ++k) v = fmaf(pw[r * top + k], pairs[(r * top + k) * D + d], v);
        rowbuf[d] = v;
        q = fmaf(v, v, q);
    }
    const float rr = sqrtf(block_sum(q, scratch) / (float)D + eps);
    float q2 = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = rowbuf[d] / rr * w[d];
        if (ls) v *= ls[d];
        v += xr[d];
        xr[d] = v;
        rowbuf[d] = v;
        q2 = fmaf(v, v, q2);
    }
    if (!nw) return;
    const float r2 = sqrtf(block_sum(q2, scratch) / (float)D + neps);
    TOut* hr = h + r * h_stride;
    for (int d = threadIdx.x; d < D; d += blockDim.x) hr[d] = from_f32<TOut>(rowbuf[d] / r2 * (nw[d] + noff));
}

// The join of a block that norms after the sum: with v = y[r] (+ sum_k pw[r][k] * pairs[r * top + k], the weighted results
// of a routed feed-forward's chosen experts, in the order of k; y or the pairs may be absent, and both: v = 0),
//   x[r] <- (alpha * x[r] + v) / sqrt(mean((alpha * x[r] + v)^2) + eps) * w,
// all 32-bit, in place; h (if given) gets the new x in the activation dtype, for the products that read it next.
template <typename TOut>
__global__ void __launch_bounds__(256)
post_norm_kernel(const float* y, long long y_stride, const float* pairs, const float* pw, int top, const float* __restrict__ w,
                 float alpha, float* x, long long x_stride, TOut* h, long long h_stride, int D, float eps) {
    extern __shared__ float rowbuf[];       // [D]
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch();
    const size_t r = blockIdx.x;
    float* xr = x + r * x_stride;
    float q = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float v = y ? y[r * y_stride + d] : 0.f;
        if (pairs)
            for (int k = 0; k < top; ++k) v = fmaf(pw[r * top + k], pairs[(r * top + k) * D + d], v);
        v = fmaf(alpha, xr[d], v);
        rowbuf[d] = v;
        q = fmaf(v, v, q);
    }
    const float rr = sqrtf(block_sum(q, scratch) / (float)D + eps);
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = rowbuf[d] / rr * w[d];
        xr[d] = v;
        if (h) h[r * h_stride + d] = from_f32<TOut>(v);
    }
}

}  // namespace

MLLM_EXPORT int mllm_post_norm(const float* y, long long y_stride, const float* pairs, const float* pw, int top, const float* w,
                               float alpha, float* x, long long x_stride, void* h, long long h_stride, int R, int D, float eps,
                               int h_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (D <= 0 || (size_t)D * 4 > 200 * 1024) return mllm_fail(1, "post_norm: width %d", D);
    if (pairs && (!pw || top <= 0)) return mllm_fail(1, "post_norm: pairs without their weights");
    const int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : ((D + 31) / 32) * 32);
    const size_t smem = (size_t)D * 4;
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        MLLM_CUDA(cudaFuncSetAttribute(post_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        MLLM_CUDA(cudaFuncSetAttribute(post_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    if (h && h_dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(post_norm_kernel<__nv_bfloat16>, dim3(R), dim3(threads), smem, stream, true, y, y_stride, pairs, pw,
                              top, w, alpha, x, x_stride, (__nv_bfloat16*)h, h_stride, D, eps));
    else if (!h || h_dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(post_norm_kernel<float>, dim3(R), dim3(threads), smem, stream, true, y, y_stride, pairs, pw, top, w,
                              alpha, x, x_stride, (float*)h, h_stride, D, eps));
    else
        return mllm_fail(1, "post_norm: unknown dtype code %d", h_dtype);
    return 0;
}

MLLM_EXPORT int mllm_norm_scale_add(const float* y, long long y_stride, const float* pairs, const float* pw, int top,
                                    const float* w, const float* ls, float* x, long long x_stride, const float* nw,
                                    float noff, float neps, void* h, long long h_stride, int R, int D, float eps,
                                    int h_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (D <= 0 || (size_t)D * 4 > 200 * 1024) return mllm_fail(1, "norm_scale_add: width %d", D);
    if (!y && !pairs) return mllm_fail(1, "norm_scale_add: neither a result nor pairs to add");
    const int threads = D >= 1024 ? 256 : (D >= 256 ? 128 : ((D + 31) / 32) * 32);
    const size_t smem = (size_t)D * 4;
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        MLLM_CUDA(cudaFuncSetAttribute(join_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        MLLM_CUDA(cudaFuncSetAttribute(join_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    if (nw && h_dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(join_kernel<__nv_bfloat16>, dim3(R), dim3(threads), smem, stream, true, y, y_stride, pairs, pw, top,
                              w, ls, x, x_stride, nw, noff, neps, (__nv_bfloat16*)h, h_stride, D, eps));
    else
        MLLM_CUDA(mllm_launch(join_kernel<float>, dim3(R), dim3(threads), smem, stream, true, y, y_stride, pairs, pw, top, w, ls,
                              x, x_stride, nw, noff, neps, (float*)h, h_stride, D, eps));
    return 0;
}

MLLM_EXPORT int mllm_rmsnorm(const float* x, long long x_stride, const int* rows, const float* w1, const float* w2,
                             void* out1, void* out2, long long out_stride, int heads, int R, int D, float eps,
                             float offset, float scale, int out_dtype, cudaStream_t stream) {
    if (R <= 0) return 0;
    if (D <= 0 || heads <= 0) return mllm_fail(1, "rmsnorm: width %d, heads %d", D, heads);
    if ((w2 == nullptr) != (out2 == nullptr)) return mllm_fail(1, "rmsnorm: the second weight and output come together");
    if (out_dtype == MLLM_F32)
        return launch<float>(x, x_stride, rows, w1, w2, out1, out2, out_stride, heads, R, D, eps, offset, scale, stream);
    if (out_dtype == MLLM_BF16)
        return launch<__nv_bfloat16>(x, x_stride, rows, w1, w2, out1, out2, out_stride, heads, R, D, eps, offset, scale,
                                     stream);
    return mllm_fail(1, "rmsnorm: unknown dtype code %d", out_dtype);
}

MLLM_EXPORT int mllm_gated_act(const void* gu, long long gu_stride, void* out, long long out_stride, int rows, int F,
                               int act, float limit, float alpha, int dtype, cudaStream_t stream) {
    if (rows <= 0 || F <= 0) return 0;
    const long long total = (long long)rows * F;
    const int grid = (int)((total + 255) / 256 < 8192 ? (total + 255) / 256 : 8192);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(gated_act_kernel<float>, dim3(grid), dim3(256), 0, stream, true, (const float*)gu, gu_stride,
                              (float*)out, out_stride, rows, F, act, limit, alpha));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(gated_act_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, true,
                              (const __nv_bfloat16*)gu, gu_stride, (__nv_bfloat16*)out, out_stride, rows, F, act, limit, alpha));
    else
        return mllm_fail(1, "gated_act: unknown dtype code %d", dtype);
    return 0;
}

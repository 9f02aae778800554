// What stands between a Q | K | V projection and attention when queries and keys are normed and rotated:
//
//   * an RMS norm over the WHOLE query projection of a token (all heads at once, H * dk numbers) and another over the
//     whole key projection (G * dk numbers), each with a plain weight vector of that length, eps inside the root
//     (either norm may be absent);
//   * a rotation of the first `rot_dims` entries of every query and key head by the angle p * f_i, p the token's
//     position and f_i a table of rot_dims / 2 frequencies.  `interleaved`: entry 2i is paired with 2i + 1; otherwise
//     entry i with i + rot_dims / 2.  The pair (u, v) becomes (u cos a - v sin a, v cos a + u sin a);
//   * `head_norm` (instead of the two norms above): after the rotation every query head and every key head is divided by
//     its own root mean square over its dk entries (eps inside the root, no weights);
//   * value mixing: with `v_first` (a row of G * dv values per token, those of an earlier layer) and a trained scalar
//     lambda the values become (1 - lambda) v + lambda v_first before they are cached; with `v_keep` the values as they
//     are cached are also written to that buffer, for the layers that mix them in later;
//   * the queries go to a buffer of their own, the keys (rows padded to `dkp` entries, the padding is never written and
//     stays zero) and the values to the token's slot in the paged cache.
//
// Sums of squares, the norm, the angle (a 32-bit product of the position and the frequency), sincosf and the rotation
// are 32-bit for both dtypes; only the results are rounded to the cache dtype.  One CTA per token; the token's query
// and key projections are kept in shared memory.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rope_kernel(const T* proj, long long ld, int q_off, int k_off, int v_off, int H, int G, int dk, int dv,
                    const float* __restrict__ qw, const float* __restrict__ kw, float eps, const float* __restrict__ freq,
                    int rot_dims, int interleaved, const int* __restrict__ positions, T* q_out, long long ldq,
                    T* __restrict__ k_pages, T* __restrict__ v_pages, int dkp, const int* __restrict__ slots, int page_size,
                    int head_norm, const T* v_first, long long ldvf, const float* __restrict__ v_lambda, T* v_keep,
                    long long ldvk) {
    extern __shared__ float row[];          // [H * dk + G * dk]; with head_norm the rotated entries and H + G factors follow
    __shared__ float scratch[33];
    pdl_wait();
    pdl_launch();
    const int t = blockIdx.x, tid = threadIdx.x;
    const int nq = H * dk, nk = G * dk;
    const T* src = proj + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    for (int i = tid; i < nq; i += blockDim.x) { const float v = to_f32(src[q_off + i]); row[i] = v; sq = fmaf(v, v, sq); }
    for (int i = tid; i < nk; i += blockDim.x) { const float v = to_f32(src[k_off + i]); row[nq + i] = v; sk = fmaf(v, v, sk); }
    float rq = 1.f, rk = 1.f;
    if (qw) rq = 1.0f / sqrtf(block_sum(sq, scratch) / (float)nq + eps);
    if (kw) rk = 1.0f / sqrtf(block_sum(sk, scratch) / (float)nk + eps);
    __syncthreads();
    const float p = (float)positions[t];
    const int slot = slots ? slots[t] : -1;
    const int half = rot_dims / 2;
    // entry d of a head: its partner, its frequency, and whether it is the first of its pair
    auto turn = [&](const float* x, const float* w, float r, int base, int d) -> float {
        const float a = x[base + d] * r * (w ? w[base + d] : 1.f);
        if (d >= rot_dims) return a;
        const int partner = interleaved ? (d ^ 1) : (d < half ? d + half : d - half);
        const bool first = interleaved ? !(d & 1) : d < half;
        const int fi = interleaved ? (d >> 1) : (d < half ? d : d - half);
        const float b = x[base + partner] * r * (w ? w[base + partner] : 1.f);
        float sn, cs;
        sincosf(p * freq[fi], &sn, &cs);
        return first ? a * cs - b * sn : a * cs + b * sn;
    };
    T* qrow = q_out + (size_t)t * ldq;
    const size_t prow = slot >= 0 ? (size_t)(slot / page_size) * G : 0;
    const int off = slot >= 0 ? slot % page_size : 0;
    if (head_norm) {
        float* rot = row + nq + nk;         // the rotated queries and keys
        float* hs = rot + nq + nk;          // 1 / rms of every query head, then of every key head
        for (int i = tid; i < nq + nk; i += blockDim.x) {
            const int j = i < nq ? i : i - nq;
            rot[i] = turn(i < nq ? row : row + nq, nullptr, 1.f, (j / dk) * dk, j % dk);
        }
        __syncthreads();
        const int warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
        for (int hd = warp; hd < H + G; hd += nwarp) {
            float ss = 0.f;
            for (int d = lane; d < dk; d += 32) { const float v = rot[hd * dk + d]; ss = fmaf(v, v, ss); }
            ss = warp_sum(ss);
            if (lane == 0) hs[hd] = 1.0f / sqrtf(ss / (float)dk + eps);
        }
        __syncthreads();
        for (int i = tid; i < nq; i += blockDim.x) qrow[i] = from_f32<T>(rot[i] * hs[i / dk]);
        if (slot >= 0)
            for (int i = tid; i < nk; i += blockDim.x) {
                const int g = i / dk, d = i % dk;
                k_pages[((prow + g) * page_size + off) * dkp + d] = from_f32<T>(rot[nq + i] * hs[H + g]);
            }
    } else {
        for (int i = tid; i < nq; i += blockDim.x) qrow[i] = from_f32<T>(turn(row, qw, rq, (i / dk) * dk, i % dk));
        if (slot >= 0)
            for (int i = tid; i < nk; i += blockDim.x) {
                const int g = i / dk, d = i % dk;
                k_pages[((prow + g) * page_size + off) * dkp + d] = from_f32<T>(turn(row + nq, kw, rk, g * dk, d));
            }
    }
    if (slot >= 0 || v_keep) {
        const float lam = v_first ? v_lambda[0] : 0.f;
        for (int i = tid; i < G * dv; i += blockDim.x) {
            const int g = i / dv, d = i % dv;
            T val = src[v_off + i];
            if (v_first) val = from_f32<T>((1.0f - lam) * to_f32(val) + lam * to_f32(v_first[(size_t)t * ldvf + i]));
            if (v_keep) v_keep[(size_t)t * ldvk + i] = val;
            if (slot >= 0) v_pages[((prow + g) * page_size + off) * dv + d] = val;
        }
    }
}

}  // namespace

// proj [T, ...] holds the token's queries at column q_off (H * dk), keys at k_off (G * dk), values at v_off (G * dv).
// qw / kw: norm weights or null; freq: rot_dims / 2 frequencies (null when rot_dims is 0); slots: the tokens' cache
// slots or null (nothing is written to the cache then).  head_norm: 1 for the per-head norm after the rotation (qw and kw
// must then be null).  v_first [T, G * dv] with lambda (one float on the device), v_keep [T, G * dv]: value mixing, or null.
MLLM_EXPORT int mllm_qk_norm_rope(const void* proj, long long ld, int q_off, int k_off, int v_off, int H, int G, int dk, int dv,
                                  const float* qw, const float* kw, float eps, const float* freq, int rot_dims, int interleaved,
                                  const int* positions, void* q_out, long long ldq, void* k_pages, void* v_pages, int dkp,
                                  const int* slots, int page_size, int head_norm, const void* v_first, long long ldvf,
                                  const float* v_lambda, void* v_keep, long long ldvk, int T, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (head_norm && (qw || kw)) return mllm_fail(1, "qk_norm_rope: the per-head norm takes no weights");
    if (v_first && !v_lambda) return mllm_fail(1, "qk_norm_rope: values to mix in without their factor");
    if (H <= 0 || G <= 0 || dk <= 0 || dv <= 0 || dkp < dk)
        return mllm_fail(1, "qk_norm_rope: %d / %d heads of %d (rows of %d) and %d", H, G, dk, dkp, dv);
    if (rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > dk || (rot_dims > 0 && !freq))
        return mllm_fail(1, "qk_norm_rope: %d rotated entries of %d", rot_dims, dk);
    if (slots && (!k_pages || !v_pages || page_size <= 0)) return mllm_fail(1, "qk_norm_rope: cache slots without pages");
    const size_t smem = sizeof(float) * (head_norm ? 2 * ((size_t)H * dk + (size_t)G * dk) + H + G : (size_t)H * dk + (size_t)G * dk);
    if (smem > 200 * 1024) return mllm_fail(1, "qk_norm_rope: projections of %d + %d entries do not fit shared memory", H * dk, G * dk);
    if (dtype == MLLM_F32) {
        if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(qk_norm_rope_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MLLM_CUDA(mllm_launch(qk_norm_rope_kernel<float>, dim3(T), dim3(256), smem, stream, true, (const float*)proj, ld, q_off,
                              k_off, v_off, H, G, dk, dv, qw, kw, eps, freq, rot_dims, interleaved, positions, (float*)q_out, ldq,
                              (float*)k_pages, (float*)v_pages, dkp, slots, page_size, head_norm, (const float*)v_first, ldvf,
                              v_lambda, (float*)v_keep, ldvk));
    } else if (dtype == MLLM_BF16) {
        using bf = __nv_bfloat16;
        if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(qk_norm_rope_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        MLLM_CUDA(mllm_launch(qk_norm_rope_kernel<bf>, dim3(T), dim3(256), smem, stream, true, (const bf*)proj, ld, q_off, k_off,
                              v_off, H, G, dk, dv, qw, kw, eps, freq, rot_dims, interleaved, positions, (bf*)q_out, ldq,
                              (bf*)k_pages, (bf*)v_pages, dkp, slots, page_size, head_norm, (const bf*)v_first, ldvf, v_lambda,
                              (bf*)v_keep, ldvk));
    } else {
        return mllm_fail(1, "qk_norm_rope: unknown dtype code %d", dtype);
    }
    return 0;
}

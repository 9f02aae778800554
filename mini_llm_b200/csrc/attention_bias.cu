// Causal softmax attention over the paged cache with three things the plain kernels do not have:
//   * keys and values of different row sizes (dk for queries and keys, dv for values and outputs);
//   * an additive score bias that depends on the head and on the distance i - j only, given as a table
//     dist_bias[head][distance] (a logarithmic or linear distance penalty, say);
//   * a factor on the query that depends on its position only, given as a table q_scale[position]
//     (a query "temperature" that grows with the context).
// score(i, j) = (q_i . k_j) * scale * q_scale[i] + dist_bias[h][i - j] for j <= i (and j > i - window when a
// window is set, and j >= floor(i / chunk) * chunk when a chunk is set: block b is positions [b * chunk, (b + 1) * chunk)
// of the request and a query sees only keys of its own block); softmax over the visible keys, with exp(sink[h])
// added to the denominator when a sink is given (a scalar per head: in the online softmax it is the starting maximum
// with weight 1 and a value row of zeros); out_i = out_scale * sum_j p_ij v_j.
// Two more terms that a design may ask for: a cap on the scaled product before any bias is added, s <- c * tanh(s / c)
// (`softcap` c > 0), and a linear distance penalty slope_h * (i - j) taken off the score (`slopes`, a number per head;
// the product of the slope and the distance is taken in 32-bit in the kernel, so it needs no table and no bound on the
// context).
// Either table, the slopes, the cap, the window, the chunk and the sink may be absent.
// Scores, biases, softmax and the weighted sum are 32-bit (expf, not the fast intrinsic) for both cache dtypes.
//
// Four kernels (the fourth, `mma`, is described where it stands).  `simt`: one warp per (token, head), 32 keys at a time: any step, and the plain twin of the
// others.  `tiled`: 64 queries x 32 keys per CTA and head for prompt portions: queries in shared memory, a key
// tile staged transposed and a value tile as it is, 2 x 4 scores and 2 x dv/8 outputs per thread.  `split`: single
// tokens (decode): the keys of a token are cut into splits of 256 starting at multiples of 256 from position 0, a
// CTA takes one split for up to four query heads that share a key/value head (rows staged once in shared memory),
// the partial (o, m, l) of the splits are merged in split order by a second kernel.  Key chunks and tiles start at multiples of 32 from position 0 in all three, so a token's
// sums run in an order that depends on its position only, not on how the step was cut or batched.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_D = 256;          // largest dk and dv

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f) {   // 8 consecutive elements (bfloat16) or 4 + 4 (float)
    if constexpr (sizeof(T) == 4) {
        const float4 a = *reinterpret_cast<const float4*>(p);
        const float4 b = *reinterpret_cast<const float4*>(p + 4);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(b2[i]); f[2 * i + 1] = __high2float(b2[i]); }
    }
}

struct BiasArgs {
    const float* dist_bias;     // [H][n_dist] or null
    int n_dist;
    const float* q_scale;       // [n_pos] or null
    float scale, out_scale;
    int window;
    int chunk;                  // > 0: keys before floor(p / chunk) * chunk are not seen
    const float* sink;          // [H] or null: exp(sink[h]) joins the softmax denominator
    float softcap;              // > 0: the scaled product s becomes softcap * tanh(s / softcap) before the biases
    const float* slopes;        // [H] or null: slopes[h] * (i - j) is taken off the score
};

// the cap on a scaled product (before any bias)
__device__ __forceinline__ float capped(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

// first key position that the query at position p sees
__device__ __forceinline__ int first_visible(const BiasArgs& a, int p) {
    int first = 0;
    if (a.window > 0 && p - a.window + 1 > 0) first = p - a.window + 1;
    if (a.chunk > 0) first = max(first, (p / a.chunk) * a.chunk);
    return first;
}

// One warp walks the keys [k_lo, k_hi] (inclusive, absolute positions) of one (token, head) in chunks of 32 that
// start at multiples of 32, and leaves the online-softmax state: acc (lane d holds dims d, d+32, ...), m, l.
template <typename T>
__device__ __forceinline__ void warp_walk(const float* qs, const T* k_pages, const T* v_pages, const int* bt, int p, int h,
                                          int hk, int Hkv, int dk, int dv, int page_size, int k_lo, int k_hi,
                                          const BiasArgs& a, float qf, float* acc, float& m, float& l) {
    const int lane = threadIdx.x & 31;
    constexpr int NACC = MAX_D / 32;
    const float* brow = a.dist_bias ? a.dist_bias + (size_t)h * a.n_dist : nullptr;
    const float slope = a.slopes ? a.slopes[h] : 0.f;
    for (int c0 = (k_lo / 32) * 32; c0 <= k_hi; c0 += 32) {
        const int kp = c0 + lane;
        const bool valid = kp >= k_lo && kp <= k_hi;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[kp / page_size];
            const T* kr = k_pages + (((size_t)page * Hkv + hk) * page_size + kp % page_size) * dk;
            float dot = 0.f;
            for (int d = 0; d < dk; d += 8) {
                float kv[8];
                load8(kr + d, kv);
#pragma unroll
                for (int i = 0; i < 8; ++i) dot = fmaf(qs[d + i], kv[i], dot);
            }
            s = capped(dot * qf, a.softcap);
            if (brow) s += brow[p - kp];
            if (a.slopes) s -= slope * (float)(p - kp);
        }
        const float m_new = fmaxf(m, warp_max(s));
        if (m_new == -INFINITY) continue;                 // no key of the chunk is in the range (uniform)
        const float alpha = expf(m - m_new);
        const float pr = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const int j0 = max(0, k_lo - c0), j1 = min(32, k_hi - c0 + 1);
        for (int j = j0; j < j1; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const int kpj = c0 + j;
            const int page = bt[kpj / page_size];
            const T* vr = v_pages + (((size_t)page * Hkv + hk) * page_size + kpj % page_size) * dv;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_bias_simt_kernel(const T* q, long long q_stride, const T* k_pages, const T* v_pages,
                           const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_seq,
                           const int* __restrict__ positions, T* __restrict__ out, long long out_stride, int T_tokens,
                           int H, int Hkv, int dkq, int dk, int dv, int page_size, BiasArgs a) {
    __shared__ float qs[WARPS][MAX_D];
    pdl_wait();
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * WARPS + warp;
    if (gw >= (long long)T_tokens * H) return;
    const int t = (int)(gw / H), h = (int)(gw % H);
    const int hk = h / (H / Hkv);
    const int seq = token_seq[t], p = positions[t];
    const int* bt = block_table + (size_t)seq * bt_stride;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * dkq;
    for (int d = lane; d < dk; d += 32) qs[warp][d] = d < dkq ? to_f32(qrow[d]) : 0.f;     // key rows are padded with zeros
    __syncwarp();
    const float qf = a.scale * (a.q_scale ? a.q_scale[p] : 1.0f);
    const int first = first_visible(a, p);
    constexpr int NACC = MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    if (a.sink) { m = a.sink[h]; l = 1.f; }
    warp_walk<T>(qs[warp], k_pages, v_pages, bt, p, h, hk, Hkv, dk, dv, page_size, first, p, a, qf, acc, m, l);
    T* orow = out + (size_t)t * out_stride + (size_t)h * dv;
    const float inv = a.out_scale / l;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

// ------------------------------------------------------------------------------------------------ decode
constexpr int SPLIT = 256;          // keys per split

// Single tokens.  grid (splits, kv heads x head chunks, tokens).  A CTA takes one split of one token's keys for HG
// (1, 2 or 4) query heads that share a key/value head, so a key or value row is fetched once for all of them.  The
// split is walked in tiles of 32 * KS * NT keys (KS = 4 / HG warps per head; NT chunks per warp: the whole split at once
// where shared memory allows) that are staged in shared memory with 16-byte loads (all loads of a burst before any
// store); warp w takes head w % HG and the chunks w / HG, w / HG + KS, ...: its lanes are the 32 keys for the scores (a
// row of K per lane, the query broadcast) and 32 value columns at a time for the weighted sum.  Chunks cover 32
// consecutive positions starting at multiples of 32 from position 0.
// Partial results: part_o [T][H][splits][dv], part_ml [T][H][splits][2]; a split without visible keys writes l = 0.
template <typename T>
__global__ void __launch_bounds__(128)
attention_bias_split_kernel(const T* q, long long q_stride, const T* k_pages, const T* v_pages,
                            const int* __restrict__ block_table, int bt_stride, const int* __restrict__ token_seq,
                            const int* __restrict__ positions, float* __restrict__ part_o, float* __restrict__ part_ml,
                            int H, int Hkv, int dkq, int dk, int dv, int page_size, int HG, int KS, int NT, BiasArgs a) {
    extern __shared__ __align__(16) unsigned char smraw[];
    constexpr int VEC = 16 / sizeof(T);
    const int krow = dk + VEC;                                  // elements per staged key row: 16 bytes of padding
    const int tile = 32 * KS * NT;                              // keys staged at a time: NT chunks of 32 per warp
    T* Ks = reinterpret_cast<T*>(smraw);                        // [tile][dk + VEC]
    T* Vs = Ks + (size_t)tile * krow;                           // [tile][dv]
    float* qs = reinterpret_cast<float*>(Vs + (((size_t)tile * dv + VEC - 1) / VEC) * VEC);   // [HG][dk]
    float* so = qs + HG * dk;                                   // [warps][dv] at the end
    float* sml = so + 4 * dv;                                   // [warps][2]
    pdl_wait();
    pdl_launch();
    const int split = blockIdx.x, nsplit = gridDim.x, t = blockIdx.z;
    const int R = H / Hkv, chunks = (R + HG - 1) / HG;
    const int hk = blockIdx.y / chunks, h0 = hk * R + (blockIdx.y % chunks) * HG;
    const int nh = min(HG, hk * R + R - h0);                    // heads this CTA really has
    const int tid = threadIdx.x, nthreads = blockDim.x, warp = tid >> 5, lane = tid & 31;
    const int wh = warp % HG, wk = warp / HG;                   // this warp's head and key sub-tile
    const int h = h0 + wh;
    const bool live = wh < nh;
    const int seq = token_seq[t], p = positions[t];
    const int first = first_visible(a, p);
    const int s_lo = max(first, split * SPLIT), s_hi = min(p, split * SPLIT + SPLIT - 1);
    if (s_lo > s_hi) {                                          // uniform over the CTA
        if (tid < nh) { const size_t pi = ((size_t)t * H + h0 + tid) * nsplit + split; part_ml[pi * 2] = -INFINITY; part_ml[pi * 2 + 1] = 0.f; }
        return;
    }
    const int* bt = block_table + (size_t)seq * bt_stride;
    for (int i = tid; i < HG * dk; i += nthreads) {
        const int hh = i / dk, d = i % dk;
        qs[i] = (hh < nh && d < dkq) ? to_f32(q[(size_t)t * q_stride + (size_t)(h0 + hh) * dkq + d]) : 0.f;
    }
    const float qf = a.scale * (a.q_scale ? a.q_scale[p] : 1.0f);
    const float* brow = (a.dist_bias && live) ? a.dist_bias + (size_t)h * a.n_dist : nullptr;
    const float slope = (a.slopes && live) ? a.slopes[h] : 0.f;
    constexpr int NACC = MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int kpieces = dk / VEC;
    const int vpieces = (dv % VEC == 0 && ((uintptr_t)v_pages % 16) == 0) ? dv / VEC : 0;   // 0: value rows are copied by element

    for (int base = (s_lo / tile) * tile; base <= s_hi; base += tile) {
        __syncthreads();                                        // the tile before is no longer read; qs is complete
        constexpr int LD = 4;
        for (int i0 = tid; i0 < tile * kpieces; i0 += nthreads * LD) {
            uint4 r[LD];
#pragma unroll
            for (int u = 0; u < LD; ++u) {
                const int i = i0 + u * nthreads, key = i / kpieces, piece = i % kpieces, kp = base + key;
                r[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i < tile * kpieces && kp >= s_lo && kp <= s_hi)
                    r[u] = *reinterpret_cast<const uint4*>(k_pages + (((size_t)bt[kp / page_size] * Hkv + hk) * page_size + kp % page_size) * dk + piece * VEC);
            }
#pragma unroll
            for (int u = 0; u < LD; ++u) {
                const int i = i0 + u * nthreads;
                if (i < tile * kpieces) *reinterpret_cast<uint4*>(Ks + (size_t)(i / kpieces) * krow + (i % kpieces) * VEC) = r[u];
            }
        }
        if (vpieces) {
            for (int i0 = tid; i0 < tile * vpieces; i0 += nthreads * LD) {
                uint4 r[LD];
#pragma unroll
                for (int u = 0; u < LD; ++u) {
                    const int i = i0 + u * nthreads, key = i / vpieces, piece = i % vpieces, kp = base + key;
                    r[u] = make_uint4(0u, 0u, 0u, 0u);
                    if (i < tile * vpieces && kp >= s_lo && kp <= s_hi)
                        r[u] = *reinterpret_cast<const uint4*>(v_pages + (((size_t)bt[kp / page_size] * Hkv + hk) * page_size + kp % page_size) * dv + piece * VEC);
                }
#pragma unroll
                for (int u = 0; u < LD; ++u) {
                    const int i = i0 + u * nthreads;
                    if (i < tile * vpieces) *reinterpret_cast<uint4*>(Vs + (size_t)(i / vpieces) * dv + (i % vpieces) * VEC) = r[u];
                }
            }
        } else {
            for (int i = tid; i < tile * dv; i += nthreads) {
                const int key = i / dv, d = i % dv, kp = base + key;
                T val = from_f32<T>(0.f);
                if (kp >= s_lo && kp <= s_hi)
                    val = v_pages[(((size_t)bt[kp / page_size] * Hkv + hk) * page_size + kp % page_size) * dv + d];
                Vs[(size_t)key * dv + d] = val;
            }
        }
        __syncthreads();
        for (int it = 0; it < NT; ++it) {
        const int ck = (it * KS + wk) * 32;                     // this warp's chunk of 32 keys within the tile
        const int c0 = base + ck;
        if (!live || c0 > s_hi || c0 + 31 < s_lo) continue;     // uniform over the warp (barriers are outside)
        const int kp = c0 + lane;
        const bool valid = kp >= s_lo && kp <= s_hi;
        const T* kr = Ks + (size_t)(ck + lane) * krow;
        const float* qh = qs + wh * dk;
        float dot = 0.f;
        for (int d = 0; d < dk; d += VEC) {
            float kv[8];
            if constexpr (sizeof(T) == 4) {
                const float4 x = *reinterpret_cast<const float4*>(kr + d);
                kv[0] = x.x; kv[1] = x.y; kv[2] = x.z; kv[3] = x.w;
            } else {
                load8(kr + d, kv);
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) dot = fmaf(qh[d + e], kv[e], dot);
        }
        float sc = -INFINITY;
        if (valid) {
            sc = capped(dot * qf, a.softcap);
            if (brow) sc += brow[p - kp];
            if (a.slopes) sc -= slope * (float)(p - kp);
        }
        const float m_new = fmaxf(m, warp_max(sc));             // at least one key of the chunk is visible
        const float alpha = expf(m - m_new);
        const float pr = valid ? expf(sc - m_new) : 0.f;
        l = l * alpha + warp_sum(pr);
        m = m_new;
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= alpha;
        const T* vt = Vs + (size_t)ck * dv;
#pragma unroll 4
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, pr, j);
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int d = lane + 32 * i;
                if (d < dv) acc[i] = fmaf(pj, to_f32(vt[(size_t)j * dv + d]), acc[i]);
            }
        }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) so[warp * dv + d] = acc[i];
    }
    if (lane == 0) { sml[warp * 2] = m; sml[warp * 2 + 1] = l; }
    __syncthreads();
    // the key sub-tiles of a head meet in sub-tile order
    for (int hh = 0; hh < nh; ++hh) {
        float mm = -INFINITY;
        for (int k = 0; k < KS; ++k)
            if (sml[(k * HG + hh) * 2 + 1] > 0.f) mm = fmaxf(mm, sml[(k * HG + hh) * 2]);
        float ll = 0.f;
        for (int k = 0; k < KS; ++k) {
            const float lw = sml[(k * HG + hh) * 2 + 1];
            if (lw > 0.f) ll += lw * expf(sml[(k * HG + hh) * 2] - mm);
        }
        const size_t pi = ((size_t)t * H + h0 + hh) * nsplit + split;
        for (int d = tid; d < dv; d += nthreads) {
            float o = 0.f;
            for (int k = 0; k < KS; ++k) {
                const float lw = sml[(k * HG + hh) * 2 + 1];
                if (lw > 0.f) o += so[(k * HG + hh) * dv + d] * expf(sml[(k * HG + hh) * 2] - mm);
            }
            part_o[pi * dv + d] = o;
        }
        if (tid == 0) { part_ml[pi * 2] = mm; part_ml[pi * 2 + 1] = ll; }
    }
}

// One warp per (token, head): out = out_scale * sum_s o_s e^(m_s - m) / sum_s l_s e^(m_s - m), in split order.
template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_bias_merge_kernel(const float* part_o, const float* part_ml, const int* __restrict__ positions,
                            T* __restrict__ out, long long out_stride, int T_tokens, int H, int dv, int nsplit,
                            float out_scale, const float* __restrict__ sink) {
    pdl_wait();
    pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long gw = (long long)blockIdx.x * WARPS + warp;
    if (gw >= (long long)T_tokens * H) return;
    const int t = (int)(gw / H), h = (int)(gw % H);
    const int used = min(nsplit, positions[t] / SPLIT + 1);
    const size_t base = ((size_t)t * H + h) * nsplit;
    float mm = sink ? sink[h] : -INFINITY;
    for (int s = 0; s < used; ++s)
        if (part_ml[(base + s) * 2 + 1] > 0.f) mm = fmaxf(mm, part_ml[(base + s) * 2]);
    float ll = sink ? expf(sink[h] - mm) : 0.f;              // the sink's term, taken before the splits'
    constexpr int NACC = MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    for (int s = 0; s < used; ++s) {
        const float ls = part_ml[(base + s) * 2 + 1];
        if (!(ls > 0.f)) continue;
        const float f = expf(part_ml[(base + s) * 2] - mm);
        ll += ls * f;
#pragma unroll
        for (int i = 0; i < NACC; ++i) {
            const int d = lane + 32 * i;
            if (d < dv) acc[i] = fmaf(part_o[(base + s) * dv + d], f, acc[i]);
        }
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * dv;
    const float inv = out_scale / ll;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int d = lane + 32 * i;
        if (d < dv) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

// ------------------------------------------------------------------------------------------------ prompt portions
constexpr int BQ = 64, BK = 32, THREADS = 256;

// grid (H, tiles).  A tile is up to 64 consecutive new tokens of one request (request, first flat token, rows).
template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_bias_tiled_kernel(const T* q, long long q_stride, const T* k_pages, const T* v_pages,
                            const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tiles,
                            const int* __restrict__ positions, T* __restrict__ out, long long out_stride, int H, int Hkv,
                            int dkq, int dk, int dv, int page_size, BiasArgs a) {
    extern __shared__ float sm[];
    const int qrow = dk + 1;
    float* Qs = sm;                         // [BQ][dk+1]   queries times scale times their position's factor
    float* Kt = Qs + BQ * qrow;             // [dk][BK]
    float* Vs = Kt + dk * BK;               // [BK][dv]
    float* Ps = Vs + BK * dv;               // [BQ][BK+1]
    float* Bs = Ps + BQ * (BK + 1);         // [BQ+BK]      the head's bias at the distances this tile pair can have
    pdl_wait();
    pdl_launch();
    const int tile = blockIdx.y, h = blockIdx.x;
    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0], pos_max = pos0 + rows - 1;
    const int hk = h / (H / Hkv);
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, ty = tid >> 3, tx = tid & 7;          // rows 2ty, 2ty+1; keys 4tx..4tx+3; dims tx + 8i
    const int first_key = first_visible(a, pos0);           // of the tile's first row: later rows see no earlier key
    const float* brow = a.dist_bias ? a.dist_bias + (size_t)h * a.n_dist : nullptr;
    const float slope = a.slopes ? a.slopes[h] : 0.f;
    const bool biased = brow || a.slopes;

    for (int i = tid; i < BQ * dk; i += THREADS) {
        const int r = i / dk, d = i % dk;
        float v = 0.f;
        if (r < rows && d < dkq) {
            const float qf = a.scale * (a.q_scale ? a.q_scale[pos0 + r] : 1.0f);
            v = to_f32(q[(size_t)(tok0 + r) * q_stride + (size_t)h * dkq + d]) * qf;
        }
        Qs[r * qrow + d] = v;
    }
    constexpr int MAXI = MAX_D / 8;
    float o[2][MAXI];
#pragma unroll
    for (int i = 0; i < MAXI; ++i) { o[0][i] = 0.f; o[1][i] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    if (a.sink) { m_run[0] = m_run[1] = a.sink[h]; l_run[0] = l_run[1] = 1.f; }
    const int nd = (dv + 7) / 8;
    const int q0 = pos0 + 2 * ty;           // absolute position of this thread's first row
    constexpr int VEC = 16 / sizeof(T);

    for (int j = first_key / BK; j <= pos_max / BK; ++j) {
        __syncthreads();                    // the previous tile is no longer read (and Qs is complete)
        const int kpieces = dk / VEC;
        for (int i = tid; i < BK * kpieces; i += THREADS) {
            const int key = i % BK, piece = i / BK;
            const int kp = j * BK + key;
            float kf[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) kf[e] = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                const T* src = k_pages + (((size_t)page * Hkv + hk) * page_size + kp % page_size) * dk + piece * VEC;
                if constexpr (sizeof(T) == 4) {
                    const float4 x = *reinterpret_cast<const float4*>(src);
                    kf[0] = x.x; kf[1] = x.y; kf[2] = x.z; kf[3] = x.w;
                } else {
                    load8(src, kf);
                }
            }
#pragma unroll
            for (int e = 0; e < VEC; ++e) Kt[(piece * VEC + e) * BK + key] = kf[e];
        }
        for (int i = tid; i < BK * dv; i += THREADS) {
            const int key = i / dv, d = i % dv;
            const int kp = j * BK + key;
            float v = 0.f;
            if (kp <= pos_max && kp >= first_key) {
                const int page = bt[kp / page_size];
                v = to_f32(v_pages[(((size_t)page * Hkv + hk) * page_size + kp % page_size) * dv + d]);
            }
            Vs[key * dv + d] = v;
        }
        // distances between this query tile and this key tile: pos0 - (j*BK + BK-1) .. pos_max - j*BK
        const int dist0 = pos0 - (j * BK + BK - 1);
        if (biased)
            for (int i = tid; i < BQ + BK; i += THREADS) {
                const int dist = dist0 + i;
                float b = (brow && dist >= 0 && dist < a.n_dist) ? brow[dist] : 0.f;
                if (a.slopes && dist >= 0) b -= slope * (float)dist;
                Bs[i] = b;
            }
        __syncthreads();
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        const float* qa = Qs + (2 * ty) * qrow;
        const float* qb = qa + qrow;
        for (int d = 0; d < dk; ++d) {
            const float4 kv = *reinterpret_cast<const float4*>(Kt + d * BK + 4 * tx);
            const float x = qa[d], y = qb[d];
            s[0][0] = fmaf(x, kv.x, s[0][0]); s[0][1] = fmaf(x, kv.y, s[0][1]);
            s[0][2] = fmaf(x, kv.z, s[0][2]); s[0][3] = fmaf(x, kv.w, s[0][3]);
            s[1][0] = fmaf(y, kv.x, s[1][0]); s[1][1] = fmaf(y, kv.y, s[1][1]);
            s[1][2] = fmaf(y, kv.z, s[1][2]); s[1][3] = fmaf(y, kv.w, s[1][3]);
        }
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int qp = q0 + r;
            float mx = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int kp = j * BK + 4 * tx + c;
                const bool vis = kp <= qp && qp <= pos_max && kp >= first_visible(a, qp);
                float sc = capped(s[r][c], a.softcap);
                if (biased && vis) sc += Bs[qp - kp - dist0];
                s[r][c] = vis ? sc : -INFINITY;
                mx = fmaxf(mx, s[r][c]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
            const float m_new = fmaxf(m_run[r], mx);
            const float muse = m_new == -INFINITY ? 0.f : m_new;
            alpha[r] = expf(m_run[r] - muse);
            float rs = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const float p = expf(s[r][c] - muse);
                Ps[(2 * ty + r) * (BK + 1) + 4 * tx + c] = p;
                rs += p;
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            rs += __shfl_xor_sync(0xffffffffu, rs, 4);
            l_run[r] = l_run[r] * alpha[r] + rs;
            m_run[r] = m_new;
        }
        __syncwarp();                       // a row's 8 threads are lanes of one warp: its p values are in place
#pragma unroll
        for (int i = 0; i < MAXI; ++i) {
            if (i < nd) { o[0][i] *= alpha[0]; o[1][i] *= alpha[1]; }
        }
        const float* pa = Ps + (2 * ty) * (BK + 1);
        const float* pb = pa + (BK + 1);
        for (int key = 0; key < BK; ++key) {
            const float p0 = pa[key], p1 = pb[key];
            const float* vr = Vs + key * dv + tx;
#pragma unroll
            for (int i = 0; i < MAXI; ++i) {
                if (i < nd && tx + 8 * i < dv) {
                    const float v = vr[8 * i];
                    o[0][i] = fmaf(p0, v, o[0][i]);
                    o[1][i] = fmaf(p1, v, o[1][i]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = 2 * ty + r;
        if (row >= rows) continue;
        const float inv = a.out_scale / l_run[r];
        T* orow = out + (size_t)(tok0 + row) * out_stride + (size_t)h * dv;
#pragma unroll
        for (int i = 0; i < MAXI; ++i)
            if (i < nd && tx + 8 * i < dv) orow[tx + 8 * i] = from_f32<T>(o[r][i] * inv);
    }
}

// ------------------------------------------------------------------------------------------------ prompt portions, bfloat16
// The same attention on tensor cores (mma.sync m16n8k16, bfloat16 operands, 32-bit accumulators) for key and value
// sizes that are multiples of 16 up to 128.  A CTA of four warps takes one tile of up to 64 new tokens and one head;
// a warp owns 16 query rows.  Key tile j covers the absolute positions [64j, 64j + 64).  Keys and values come into
// shared memory by cp.async (rows nobody sees are zero-filled), the next tile's while the current one is used.
// S = Q K^T is accumulated in 32-bit; the query's factor, the scale and the distance bias are applied to the 32-bit
// sums; the online softmax is 32-bit (scores in units of ln 2 and ex2.approx); the weights go into the second product as p = hi + lo, two bfloat16
// terms, so that they keep about 16 bits; the output sums are 32-bit.
constexpr int MQ = 64, MK = 64, MMAX = 128;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void ldsm_x4(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t* r, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = valid ? 16 : 0;                                // 0 bytes read: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float ex2(float x) {                   // 2^x in one instruction; 2^(-inf) = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// NO: value tiles of 8 columns the kernel is compiled for (4, 8 or 16: value sizes up to 32, 64, 128)
template <int NO>
__global__ void __launch_bounds__(128)
attention_bias_mma_kernel(const __nv_bfloat16* q, long long q_stride, const __nv_bfloat16* k_pages, const __nv_bfloat16* v_pages,
                          const int* __restrict__ block_table, int bt_stride, const int* __restrict__ tiles,
                          const int* __restrict__ positions, __nv_bfloat16* __restrict__ out, long long out_stride, int H,
                          int Hkv, int dk, int dv, int page_size, BiasArgs a) {
    using bf = __nv_bfloat16;
    extern __shared__ __align__(16) unsigned char smraw[];
    const int qrow = dk + 8, krow = dk + 8, vrow = dv + 8;       // 16 bytes of padding: ldmatrix rows fall on different banks
    bf* Qs = reinterpret_cast<bf*>(smraw);                       // [MQ][dk+8]
    bf* Ks = Qs + MQ * qrow;                                     // [2][MK][dk+8]
    bf* Vs = Ks + 2 * MK * krow;                                 // [2][MK][dv+8]
    float* Bs = reinterpret_cast<float*>(Vs + 2 * MK * vrow);    // [2][MQ+MK] the head's bias at the distances of a tile pair
    pdl_wait();
    pdl_launch();
    const int tile = blockIdx.y, h = blockIdx.x;
    const int seq = tiles[tile * 3], tok0 = tiles[tile * 3 + 1], rows = tiles[tile * 3 + 2];
    const int pos0 = positions[tok0], pos_max = pos0 + rows - 1;
    const int hk = h / (H / Hkv);
    const int* bt = block_table + (size_t)seq * bt_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int first_key = first_visible(a, pos0);
    const float* brow = a.dist_bias ? a.dist_bias + (size_t)h * a.n_dist : nullptr;
    const float slope = a.slopes ? a.slopes[h] : 0.f;
    const bool biased = brow || a.slopes;
    const int kp8 = dk / 8, vp8 = dv / 8;

    // Which pieces of a tile this thread copies: the same (key, piece) pairs for every tile, so the divisions are
    // made once.  A thread copies up to MMAX / 16 pieces of keys and as many of values per tile.
    constexpr int SU = MMAX / 16;
    int k_kp[SU], v_kp[SU];                                      // key | piece << 8, or -1
#pragma unroll
    for (int u = 0; u < SU; ++u) {
        const int i = tid + u * 128;
        k_kp[u] = i < MK * kp8 ? (i / kp8) | ((i % kp8) << 8) : -1;
        v_kp[u] = i < MK * vp8 ? (i / vp8) | ((i % vp8) << 8) : -1;
    }
    const int ps_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;    // pages of a power of two: shifts
    auto row_of = [&](int kp) -> size_t {                        // first element of key position kp's row, in rows
        const int pg = ps_shift >= 0 ? kp >> ps_shift : kp / page_size;
        const int off = ps_shift >= 0 ? kp & (page_size - 1) : kp % page_size;
        return ((size_t)bt[pg] * Hkv + hk) * page_size + off;
    };
    auto stage = [&](int j, int buf) {                           // key tile j into buffer buf
        bf* kd = Ks + buf * MK * krow;
        bf* vd = Vs + buf * MK * vrow;
#pragma unroll
        for (int u = 0; u < SU; ++u) {
            if (k_kp[u] >= 0) {
                const int key = k_kp[u] & 255, piece = k_kp[u] >> 8, kp = j * MK + key;
                const bool ok = kp <= pos_max && kp >= first_key;
                cp_async16(kd + key * krow + piece * 8, ok ? k_pages + row_of(kp) * dk + piece * 8 : k_pages, ok);
            }
        }
#pragma unroll
        for (int u = 0; u < SU; ++u) {
            if (v_kp[u] >= 0) {
                const int key = v_kp[u] & 255, piece = v_kp[u] >> 8, kp = j * MK + key;
                const bool ok = kp <= pos_max && kp >= first_key;
                cp_async16(vd + key * vrow + piece * 8, ok ? v_pages + row_of(kp) * dv + piece * 8 : v_pages, ok);
            }
        }
        if (biased) {
            const int dist0 = pos0 - (j * MK + MK - 1);
            for (int i = tid; i < MQ + MK; i += 128) {
                const int dist = dist0 + i;
                float b = (brow && dist >= 0 && dist < a.n_dist) ? brow[dist] : 0.f;
                if (a.slopes && dist >= 0) b -= slope * (float)dist;
                Bs[buf * (MQ + MK) + i] = b * LOG2E;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    const int j_first = first_key / MK, j_last = pos_max / MK;
    for (int i = tid; i < MQ * kp8; i += 128) {                  // queries: rows beyond the tile are zero
        const int r = i / kp8, piece = i % kp8;
        cp_async16(Qs + r * qrow + piece * 8, r < rows ? q + (size_t)(tok0 + r) * q_stride + (size_t)h * dk + piece * 8 : q, r < rows);
    }
    stage(j_first, 0);

    const int r0 = warp * 16 + (lane >> 2);                      // this thread's rows: r0 and r0 + 8 of the tile
    const int qp0 = pos0 + r0, qp1 = qp0 + 8;
    // with a cap the factors carry 1 / cap and the capped score is cap * log2 e * tanh(.)
    const float unit = a.softcap > 0.f ? 1.0f / a.softcap : LOG2E;
    const float capl = a.softcap * LOG2E;
    const float qf0 = a.scale * unit * ((a.q_scale && r0 < rows) ? a.q_scale[qp0] : 1.0f);
    const float qf1 = a.scale * unit * ((a.q_scale && r0 + 8 < rows) ? a.q_scale[qp1] : 1.0f);
    float o[NO][4];
#pragma unroll
    for (int i = 0; i < NO; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    if (a.sink) {                                                // in units of ln 2 like the scores; one thread of a row's quad carries its weight
        m0 = m1 = a.sink[h] * LOG2E;
        l0 = l1 = (lane & 3) == 0 ? 1.f : 0.f;
    }
    const int nvt = dv / 8;

    for (int j = j_first; j <= j_last; ++j) {
        const int buf = (j - j_first) & 1;
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();                                         // tile j is in; the other buffer is free
        if (j < j_last) stage(j + 1, buf ^ 1);
        const bf* kt = Ks + buf * MK * krow;
        const bf* vt = Vs + buf * MK * vrow;
        const float* bs = Bs + buf * (MQ + MK);
        if (j * MK > pos0 + warp * 16 + 15) continue;            // every key of the tile lies after this warp's rows (uniform per warp)
        float s[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n) { s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f; }
        for (int k0 = 0; k0 < dk; k0 += 16) {
            uint32_t af[4];
            ldsm_x4(af, Qs + (warp * 16 + (lane & 15)) * qrow + k0 + (lane >> 4) * 8);
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                uint32_t bfr[2];
                ldsm_x2(bfr, kt + (n * 8 + (lane & 7)) * krow + k0 + ((lane >> 3) & 1) * 8);
                mma_bf16(s[n], af, bfr);
            }
        }
        // factor, bias, mask; row maxima.  Scores are kept in units of ln 2 (the factor and the staged bias carry
        // log2 e), so that the exponentials are exp2.  A tile that every row of the warp sees whole needs no mask.
        const int dist0 = pos0 - (j * MK + MK - 1);
        const int w_lo = pos0 + warp * 16, w_hi = w_lo + 15;
        const bool whole = j * MK + MK - 1 <= w_lo && w_hi <= pos_max && (a.window <= 0 || j * MK > w_hi - a.window) &&
                           (a.chunk <= 0 || j * MK >= (w_hi / a.chunk) * a.chunk);
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (whole) {
            const float* b0 = bs + (qp0 - j * MK - dist0) - 2 * (lane & 3);      // bias of (row r0, key j*MK + 2*(lane&3)); keys go down
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                float x0 = s[n][0] * qf0, x1 = s[n][1] * qf0, x2 = s[n][2] * qf1, x3 = s[n][3] * qf1;
                if (a.softcap > 0.f) { x0 = capl * tanhf(x0); x1 = capl * tanhf(x1); x2 = capl * tanhf(x2); x3 = capl * tanhf(x3); }
                if (biased) {
                    x0 += b0[-n * 8]; x1 += b0[-n * 8 - 1]; x2 += b0[-n * 8 + 8]; x3 += b0[-n * 8 + 7];
                }
                s[n][0] = x0; s[n][1] = x1; s[n][2] = x2; s[n][3] = x3;
                mx0 = fmaxf(mx0, fmaxf(x0, x1));
                mx1 = fmaxf(mx1, fmaxf(x2, x3));
            }
        } else {
#pragma unroll
            for (int n = 0; n < 8; ++n) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int kp = j * MK + n * 8 + 2 * (lane & 3) + (e & 1);
                    const int qp = (e < 2) ? qp0 : qp1;
                    const bool vis = kp <= qp && qp <= pos_max && kp >= first_visible(a, qp);
                    float sc = s[n][e] * ((e < 2) ? qf0 : qf1);
                    if (a.softcap > 0.f) sc = capl * tanhf(sc);
                    if (biased && vis) sc += bs[qp - kp - dist0];
                    sc = vis ? sc : -INFINITY;
                    s[n][e] = sc;
                    if (e < 2) mx0 = fmaxf(mx0, sc); else mx1 = fmaxf(mx1, sc);
                }
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float al0 = ex2(m0 - mu0), al1 = ex2(m1 - mu1);
        m0 = mn0; m1 = mn1;
        float rs0 = 0.f, rs1 = 0.f;
        uint32_t phi[4][4], plo[4][4];                           // A fragments of p for the four 16-key steps
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float p0 = ex2(s[n][0] - mu0), p1 = ex2(s[n][1] - mu0), p2 = ex2(s[n][2] - mu1), p3 = ex2(s[n][3] - mu1);
            rs0 += p0 + p1;
            rs1 += p2 + p3;
            const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
            const int kk = n >> 1, half = (n & 1) * 2;
            phi[kk][half] = *reinterpret_cast<const uint32_t*>(&h01);
            phi[kk][half + 1] = *reinterpret_cast<const uint32_t*>(&h23);
            plo[kk][half] = pack_bf16(p0 - __low2float(h01), p1 - __high2float(h01));
            plo[kk][half + 1] = pack_bf16(p2 - __low2float(h23), p3 - __high2float(h23));
        }
        l0 = l0 * al0 + rs0;                                     // per-thread part of the row sums; the quad meets at the end
        l1 = l1 * al1 + rs1;
#pragma unroll
        for (int i = 0; i < NO; ++i) {
            if (i < nvt) { o[i][0] *= al0; o[i][1] *= al0; o[i][2] *= al1; o[i][3] *= al1; }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int i = 0; i < NO; ++i) {
                if (i < nvt) {
                    uint32_t bfr[2];
                    ldsm_x2_trans(bfr, vt + (kk * 16 + (lane & 15)) * vrow + i * 8);
                    mma_bf16(o[i], phi[kk], bfr);
                    mma_bf16(o[i], plo[kk], bfr);
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = a.out_scale / l0, inv1 = a.out_scale / l1;
#pragma unroll
    for (int i = 0; i < NO; ++i) {
        if (i < nvt) {
            const int col = i * 8 + 2 * (lane & 3);
            if (r0 < rows)
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(tok0 + r0) * out_stride + (size_t)h * dv + col) =
                    __floats2bfloat162_rn(o[i][0] * inv0, o[i][1] * inv0);
            if (r0 + 8 < rows)
                *reinterpret_cast<__nv_bfloat162*>(out + (size_t)(tok0 + r0 + 8) * out_stride + (size_t)h * dv + col) =
                    __floats2bfloat162_rn(o[i][2] * inv1, o[i][3] * inv1);
        }
    }
}

int check_sizes(int H, int Hkv, int dk, int dv, int page_size, int dtype) {
    const int vec = dtype == MLLM_F32 ? 4 : 8;
    if (dtype != MLLM_F32 && dtype != MLLM_BF16) return mllm_fail(1, "attention_bias: unknown dtype code %d", dtype);
    if (dk <= 0 || dk % 8 != 0 || dk > MAX_D)
        return mllm_fail(1, "attention_bias: key size %d is not a multiple of 8 in 8..%d", dk, MAX_D);
    if (dv <= 0 || dv > MAX_D) return mllm_fail(1, "attention_bias: value size %d is not in 1..%d", dv, MAX_D);
    (void)vec;
    if (Hkv <= 0 || H % Hkv != 0) return mllm_fail(1, "attention_bias: %d heads over %d key/value heads", H, Hkv);
    if (page_size <= 0) return mllm_fail(1, "attention_bias: page size %d", page_size);
    return 0;
}

}  // namespace

MLLM_EXPORT int mllm_attention_bias_split_keys() { return SPLIT; }

// impl: 0 simt, 1 tiled (needs tiles), 2 split (single tokens; needs part_o [T*H*nsplit*dv], part_ml [T*H*nsplit*2]),
// 3 mma (bfloat16 prompt portions on tensor cores; needs tiles).
MLLM_EXPORT int mllm_attention_bias(const void* q, long long q_stride, const void* k_pages, const void* v_pages,
                                    const int* block_table, int bt_stride, const int* token_seq, const int* positions,
                                    const int* tiles, int n_tiles, void* out, long long out_stride, float* part_o,
                                    float* part_ml, int nsplit, int T, int H, int Hkv, int dkq, int dk, int dv, int page_size,
                                    float scale, float out_scale, const float* dist_bias, int n_dist,
                                    const float* q_scale, int window, int chunk, const float* sink, float softcap,
                                    const float* slopes, int dtype, int impl, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (int rc = check_sizes(H, Hkv, dk, dv, page_size, dtype)) return rc;
    if (dkq <= 0 || dkq > dk) return mllm_fail(1, "attention_bias: queries of %d against key rows of %d", dkq, dk);
    if (window < 0 || chunk < 0) return mllm_fail(1, "attention_bias: window %d, chunk %d", window, chunk);
    if (!(softcap >= 0.f)) return mllm_fail(1, "attention_bias: a cap of %g on the scores", (double)softcap);
    BiasArgs a{dist_bias, n_dist, q_scale, scale, out_scale, window, chunk, sink, softcap, slopes};
    const long long warps = (long long)T * H;
    const long long blocks = (warps + WARPS - 1) / WARPS;
    if (blocks > 2147483647LL) return mllm_fail(1, "attention_bias: too many (token, head) pairs");
    using bf = __nv_bfloat16;
    if (impl == 0) {
        if (dtype == MLLM_F32)
            MLLM_CUDA(mllm_launch(attention_bias_simt_kernel<float>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream,
                                  true, (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages,
                                  block_table, bt_stride, token_seq, positions, (float*)out, out_stride, T, H, Hkv, dkq, dk, dv,
                                  page_size, a));
        else
            MLLM_CUDA(mllm_launch(attention_bias_simt_kernel<bf>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, true,
                                  (const bf*)q, q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride,
                                  token_seq, positions, (bf*)out, out_stride, T, H, Hkv, dkq, dk, dv, page_size, a));
        return 0;
    }
    if (impl == 1) {
        if (!tiles || n_tiles <= 0) return mllm_fail(1, "attention_bias: the tiled kernel needs the step's tile list");
        const size_t smem = sizeof(float) * ((size_t)BQ * (dk + 1) + (size_t)dk * BK + (size_t)BK * dv + BQ * (BK + 1) + BQ + BK);
        if (smem > 227 * 1024) return mllm_fail(1, "attention_bias: sizes %d / %d need %zu bytes of shared memory", dk, dv, smem);
        if (dtype == MLLM_F32) {
            MLLM_CUDA(cudaFuncSetAttribute(attention_bias_tiled_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_tiled_kernel<float>, dim3(H, n_tiles), dim3(THREADS), smem, stream, true,
                                  (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table,
                                  bt_stride, tiles, positions, (float*)out, out_stride, H, Hkv, dkq, dk, dv, page_size, a));
        } else {
            MLLM_CUDA(cudaFuncSetAttribute(attention_bias_tiled_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_tiled_kernel<bf>, dim3(H, n_tiles), dim3(THREADS), smem, stream, true,
                                  (const bf*)q, q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride,
                                  tiles, positions, (bf*)out, out_stride, H, Hkv, dkq, dk, dv, page_size, a));
        }
        return 0;
    }
    if (impl == 2) {
        if (!part_o || !part_ml || nsplit <= 0) return mllm_fail(1, "attention_bias: the split kernel needs scratch for its partial results");
        const int R = H / Hkv;
        int HG = R >= 4 ? 4 : (R >= 2 ? 2 : 1), KS = 4 / HG;
        const size_t es = dtype == MLLM_F32 ? 4 : 2, vec = 16 / es;
        auto bytes = [&](int ks) {                               // ks: chunks of 32 keys staged at a time
            const size_t tile = 32 * (size_t)ks;
            return tile * (dk + vec) * es + ((tile * dv + vec - 1) / vec) * vec * es + sizeof(float) * ((size_t)HG * dk + 4 * (size_t)dv + 8);
        };
        while (KS > 1 && bytes(KS) > 96 * 1024) KS /= 2;
        // A whole split of 256 keys staged at once (one round of loads instead of up to eight) where it fits and the grid
        // is small: with few CTAs nothing else hides the loads' latency.  In a large grid (measured at batch 64: 0.57
        // against 0.71 ms per step) small tiles win, since more CTAs fit an SM and hide each other's loads.  A warp
        // walks the same chunks in the same order either way, so the result is the same bits.
        static int sms = 0;
        if (!sms) {
            int dev = 0;
            MLLM_CUDA(cudaGetDevice(&dev));
            MLLM_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        }
        int NT = 1;
        if ((long long)nsplit * Hkv * ((R + HG - 1) / HG) * T <= 4LL * sms)
            while (32 * KS * NT * 2 <= SPLIT && bytes(KS * NT * 2) <= 96 * 1024) NT *= 2;
        const size_t smem = bytes(KS * NT);
        const int chunks = (R + HG - 1) / HG;
        if ((long long)Hkv * chunks > 65535 || T > 65535) return mllm_fail(1, "attention_bias: %d heads x %d tokens exceed the split kernel's grid", H, T);
        const dim3 grid(nsplit, Hkv * chunks, T), block(32 * HG * KS);
        if (dtype == MLLM_F32) {
            if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(attention_bias_split_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_split_kernel<float>, grid, block, smem, stream, true,
                                  (const float*)q, q_stride, (const float*)k_pages, (const float*)v_pages, block_table,
                                  bt_stride, token_seq, positions, part_o, part_ml, H, Hkv, dkq, dk, dv, page_size, HG, KS, NT, a));
            MLLM_CUDA(mllm_launch(attention_bias_merge_kernel<float>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, true,
                                  (const float*)part_o, (const float*)part_ml, positions, (float*)out, out_stride, T, H, dv,
                                  nsplit, out_scale, a.sink));
        } else {
            if (smem > 48 * 1024) MLLM_CUDA(cudaFuncSetAttribute(attention_bias_split_kernel<bf>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MLLM_CUDA(mllm_launch(attention_bias_split_kernel<bf>, grid, block, smem, stream, true,
                                  (const bf*)q, q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride,
                                  token_seq, positions, part_o, part_ml, H, Hkv, dkq, dk, dv, page_size, HG, KS, NT, a));
            MLLM_CUDA(mllm_launch(attention_bias_merge_kernel<bf>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, true,
                                  (const float*)part_o, (const float*)part_ml, positions, (bf*)out, out_stride, T, H, dv,
                                  nsplit, out_scale, a.sink));
        }
        return 0;
    }
    if (impl == 3) {
        if (!tiles || n_tiles <= 0) return mllm_fail(1, "attention_bias: the tensor-core kernel needs the step's tile list");
        if (dtype != MLLM_BF16 || dkq != dk || dk % 16 != 0 || dv % 16 != 0 || dk > MMAX || dv > MMAX || out_stride % 2 != 0 ||
            (uintptr_t)out % 4 != 0 || (uintptr_t)k_pages % 16 != 0 || (uintptr_t)v_pages % 16 != 0 || (uintptr_t)q % 16 != 0 ||
            q_stride % 8 != 0)
            return mllm_fail(1, "attention_bias: the tensor-core kernel takes bfloat16, key and value sizes that are multiples "
                                "of 16 up to %d and 16-byte aligned rows (got %d / %d)", MMAX, dk, dv);
        const size_t smem = sizeof(bf) * ((size_t)MQ * (dk + 8) + 2 * (size_t)MK * (dk + 8) + 2 * (size_t)MK * (dv + 8)) +
                            sizeof(float) * 2 * (MQ + MK);
#define MLLM_MMA(NN)                                                                                                   \
    do {                                                                                                               \
        MLLM_CUDA(cudaFuncSetAttribute(attention_bias_mma_kernel<NN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        MLLM_CUDA(mllm_launch(attention_bias_mma_kernel<NN>, dim3(H, n_tiles), dim3(128), smem, stream, true, (const bf*)q,   \
                              q_stride, (const bf*)k_pages, (const bf*)v_pages, block_table, bt_stride, tiles, positions,     \
                              (bf*)out, out_stride, H, Hkv, dk, dv, page_size, a));                                           \
    } while (0)
        if (dv <= 32) MLLM_MMA(4); else if (dv <= 64) MLLM_MMA(8); else MLLM_MMA(16);
        return 0;
    }
    return mllm_fail(1, "attention_bias: unknown implementation %d", impl);
}

// rows of src [T, heads * d] (row stride given) to their page slots in pages [num_pages, heads, page_size, d]
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
paged_write_kernel(const T* src, long long row_stride, T* __restrict__ pages, const int* __restrict__ slots, int T_tokens,
                   int heads, int d, int page_size) {
    pdl_wait();
    pdl_launch();
    const int per = heads * d;
    const long long total = (long long)T_tokens * per;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per), c = (int)(i % per);
        const int slot = slots[t];
        if (slot < 0) continue;
        const int h = c / d, e = c % d;
        pages[(((size_t)(slot / page_size) * heads + h) * page_size + slot % page_size) * d + e] = src[(size_t)t * row_stride + c];
    }
}
}  // namespace

// keys [T, heads * dk] and values [T, heads * dv] of the step to their page slots in one launch; a key row of the
// pages may be longer than dk (dkp, padded to a multiple of 8 so that rows stay 16-byte aligned): the padding is
// never written and stays zero
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
paged_write_kv_kernel(const T* k, long long k_stride, const T* v, long long v_stride, T* __restrict__ k_pages,
                      T* __restrict__ v_pages, const int* __restrict__ slots, int T_tokens, int heads, int dk, int dkp, int dv,
                      int page_size) {
    pdl_wait();
    pdl_launch();
    const int pk = heads * dk, per = heads * (dk + dv);
    const long long total = (long long)T_tokens * per;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int t = (int)(i / per), c = (int)(i % per);
        const int slot = slots[t];
        if (slot < 0) continue;
        const size_t row = (size_t)(slot / page_size) * heads;
        const int off = slot % page_size;
        if (c < pk) {
            const int h = c / dk, e = c % dk;
            k_pages[((row + h) * page_size + off) * dkp + e] = k[(size_t)t * k_stride + c];     // rows of dkp >= dk: the rest stays zero
        } else {
            const int cc = c - pk, h = cc / dv, e = cc % dv;
            v_pages[((row + h) * page_size + off) * dv + e] = v[(size_t)t * v_stride + cc];
        }
    }
}
}  // namespace

MLLM_EXPORT int mllm_paged_write_kv(const void* k, long long k_stride, const void* v, long long v_stride, void* k_pages,
                                    void* v_pages, const int* slots, int T, int heads, int dk, int dkp, int dv,
                                    int page_size, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long total = (long long)T * heads * (dk + dv);
    const int grid = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(paged_write_kv_kernel<float>, dim3(grid), dim3(256), 0, stream, true, (const float*)k, k_stride,
                              (const float*)v, v_stride, (float*)k_pages, (float*)v_pages, slots, T, heads, dk, dkp, dv, page_size));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(paged_write_kv_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, true,
                              (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v, v_stride, (__nv_bfloat16*)k_pages,
                              (__nv_bfloat16*)v_pages, slots, T, heads, dk, dkp, dv, page_size));
    else
        return mllm_fail(1, "paged_write_kv: unknown dtype code %d", dtype);
    return 0;
}

MLLM_EXPORT int mllm_paged_write(const void* src, long long row_stride, void* pages, const int* slots, int T, int heads,
                                 int d, int page_size, int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    const long long total = (long long)T * heads * d;
    const int grid = (int)((total + 255) / 256 < 4096 ? (total + 255) / 256 : 4096);
    if (dtype == MLLM_F32)
        MLLM_CUDA(mllm_launch(paged_write_kernel<float>, dim3(grid), dim3(256), 0, stream, true, (const float*)src, row_stride,
                              (float*)pages, slots, T, heads, d, page_size));
    else if (dtype == MLLM_BF16)
        MLLM_CUDA(mllm_launch(paged_write_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, true,
                              (const __nv_bfloat16*)src, row_stride, (__nv_bfloat16*)pages, slots, T, heads, d, page_size));
    else
        return mllm_fail(1, "paged_write: unknown dtype code %d", dtype);
    return 0;
}

// Grouped-query attention with a capped score, a window that keeps the first tokens, and a sink in the softmax,
// over a paged cache whose rows hold a token's key and value side by side (their sizes may differ).
//
// For the query at position p of head h (kv head h / group), over cached tokens j:
//     s_j   = cap * tanh(scale * (q . k_j) / cap)          (cap = 0: s_j = scale * (q . k_j))
//     seen  = j <= p and (p - j < window or j < keep_first) (window = 0: every j <= p)
//     out   = sum_seen exp(s_j) v_j / (exp(sink_h) + sum_seen exp(s_j))
// The sink is a learned logit per head that takes weight and gives no value (sinks null: none).
// Scores, the softmax and the weighted sum are float whatever the cache's dtype.
//
//   rope_mix_kv_write   one pass over the stacked projection [q | k | v] of the step's tokens: q and k are rotated on
//                       the first `rot` entries of each head (entry i with entry i + rot/2, angle = position * f_i formed
//                       in float), q goes to its own tensor, k and v to the token's cache row; on the way
//                       v <- (1 - lambda) v + lambda v_first when an earlier layer's values are handed in.
//   attention_sink      the attention itself, from the step's work items (kernels/attention_plan.py): an item's rows
//                       attend over its key range and, in the first split of a range, over the kept first tokens
//                       before it and the sink; splits leave (max, sum, unnormalised output) for attention_reduce.
#include "common.cuh"

enum : int { KID_ATT_SINK = 70 };

#define SINK_BK 32         // keys per tile
#define SINK_MAX_ROWS 16   // query rows (token x head of the group) per CTA, one warp each
#define SINK_MAX_D 256     // largest key size and largest value size

struct SinkWork { int seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split; };

// One CTA a token.  qkv: [tokens, row_stride] with q at 0, k at nh * dk, v at (nh + nkv) * dk.
// v_first: [tokens, vf_stride] rows of nkv * dv values (null: no mixing); lambda: one float on the device.
template <typename T>
__global__ void __launch_bounds__(256) rope_mix_kv_write_kernel(const T* qkv, int row_stride, T* __restrict__ q_out,
                                                                const float* __restrict__ inv_freq, int rot,
                                                                const int* __restrict__ positions, const int* __restrict__ slots,
                                                                T* kv_pool, const T* v_first, int vf_stride,
                                                                const float* __restrict__ lambda_ptr, int nh, int nkv, int dk, int dv,
                                                                int page_size, long long pool_rows, int* status) {
    pdl_launch_dependents();
    pdl_wait(KID_ATT_SINK);
    const int t = blockIdx.x;
    const T* row = qkv + (size_t)t * row_stride;
    const float p = (float)positions[t];
    const int half = rot / 2;
    // queries
    T* qo = q_out + (size_t)t * nh * dk;
    for (int i = threadIdx.x; i < nh * dk; i += blockDim.x) {
        const int e = i % dk;
        float v = to_f32(row[i]);
        if (e < rot) {
            const int f = e < half ? e : e - half;
            float s, c;
            sincosf(p * inv_freq[f], &s, &c);
            const float other = to_f32(row[e < half ? i + half : i - half]);
            v = e < half ? v * c - other * s : v * c + other * s;
        }
        qo[i] = from_f32<T>(v);
    }
    const int slot = slots ? slots[t] : -1;
    if (kv_pool == nullptr || slot < 0) return;
    if ((long long)slot >= pool_rows) { if (threadIdx.x == 0) atomicOr(status, 2); return; }
    const int page = slot / page_size, off = slot % page_size;
    const int w = dk + dv;
    const T* kr = row + (size_t)nh * dk;
    const T* vr = kr + (size_t)nkv * dk;
    const float lam = v_first ? *lambda_ptr : 0.f;
    const T* vf = v_first ? v_first + (size_t)t * vf_stride : nullptr;
    for (int i = threadIdx.x; i < nkv * w; i += blockDim.x) {
        const int g = i / w, e = i % w;
        T* dst = kv_pool + (((size_t)page * nkv + g) * page_size + off) * w;
        float v;
        if (e < dk) {
            v = to_f32(kr[g * dk + e]);
            if (e < rot) {
                const int f = e < half ? e : e - half;
                float s, c;
                sincosf(p * inv_freq[f], &s, &c);
                const float other = to_f32(kr[g * dk + (e < half ? e + half : e - half)]);
                v = e < half ? v * c - other * s : v * c + other * s;
            }
        } else {
            v = to_f32(vr[g * dv + e - dk]);
            if (vf) v = (1.0f - lam) * v + lam * to_f32(vf[g * dv + e - dk]);
        }
        dst[e] = from_f32<T>(v);
    }
}

PLLM_EXPORT int pllm_rope_mix_kv_write(int dtype, const void* qkv, int row_stride, void* q_out, const float* inv_freq, int rot,
                                       const int* positions, const int* slots, void* kv_pool, const void* v_first, int vf_stride,
                                       const float* lambda_ptr, int n_tokens, int nh, int nkv, int dk, int dv, int page_size,
                                       long long pool_rows, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (nh <= 0 || nkv <= 0 || dk <= 0 || dv <= 0 || page_size <= 0 || rot < 0 || rot > dk || rot % 2) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(rope_mix_kv_write_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const T*)qkv, row_stride, (T*)q_out,
                       inv_freq, rot, positions, slots, (T*)kv_pool, (const T*)v_first, vf_stride, lambda_ptr, nh, nkv, dk, dv,
                       page_size, pool_rows, status);
    });
    return launch_status();
}

// One CTA per (item, kv head, part of the group); row r of the CTA (a warp) is token r / n_heads of the item and
// head head0 + r % n_heads.  Keys come in tiles of 32 through shared memory (as floats); a lane scores one key of
// the tile, then the lanes share out the value's entries.
template <typename T>
__global__ void attention_sink_kernel(const T* q,                 // [tokens, nh, dk]        (written just before: no __restrict__)
                                      const T* kv_pool,           // [pages, nkv, page_size, dk + dv]
                                      const int* __restrict__ block_tables, const SinkWork* __restrict__ work,
                                      const int* __restrict__ n_work_ptr, T* __restrict__ out,   // [tokens, nh, dv]
                                      float* __restrict__ part_o, float* __restrict__ part_ml,
                                      const float* __restrict__ sinks, int nh, int nkv, int dk, int dv, int page_size, int n_pages,
                                      int table_width, int window, int keep_first, float scale, float cap, int heads_per_cta,
                                      int* status) {
    pdl_launch_dependents();
    pdl_wait(KID_ATT_SINK);
    if ((int)blockIdx.x >= *n_work_ptr) return;
    const SinkWork w = work[blockIdx.x];
    const int group = nh / nkv;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    const int kh = blockIdx.y / gparts;
    const int head0 = kh * group + (blockIdx.y % gparts) * heads_per_cta;
    const int n_heads = min(heads_per_cta, kh * group + group - head0);
    const int rows = w.q_count * n_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int dkp = dk + 4, dvp = dv + 4;     // padded rows: float4 reads across keys without bank conflicts

    extern __shared__ float smem[];
    float* q_s = smem;                                   // [SINK_MAX_ROWS][dk]
    float* k_s = q_s + SINK_MAX_ROWS * dk;               // [SINK_BK][dkp]
    float* v_s = k_s + SINK_BK * dkp;                    // [SINK_BK][dvp]
    __shared__ int page_s[SINK_BK];

    const bool active = warp < rows;
    const int tq = active ? warp / n_heads : 0;
    const int head = active ? head0 + warp % n_heads : head0;
    const int pos = w.q_pos0 + tq;
    if (active) {
        const T* qr = q + ((size_t)(w.q_token0 + tq) * nh + head) * dk;
        for (int e = lane; e < dk; e += 32) q_s[warp * dk + e] = to_f32(qr[e]);
    }
    const bool first_split = (w.split & 0xffff) == 0;    // (an item that is not split has 0 here)
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;

    float m = -CUDART_INF_F, l = 0.f;
    float acc[SINK_MAX_D / 32];
#pragma unroll
    for (int k = 0; k < SINK_MAX_D / 32; k++) acc[k] = 0.f;

    constexpr int N = Vec16<T>::N;
    const int wrow = dk + dv;
    const bool vec = dk % N == 0 && dv % N == 0;
    const int* table = block_tables + (size_t)w.seg * table_width;

    // two ranges of keys: the kept first tokens that lie before the item's range (first split only), then the range
    for (int range = 0; range < 2; range++) {
        const int r_begin = range == 0 ? 0 : w.kv_begin;
        const int r_end = range == 0 ? (first_split && window > 0 ? min(keep_first, w.kv_begin) : 0) : w.kv_end;
        for (int kv0 = r_begin; kv0 < r_end; kv0 += SINK_BK) {
            __syncthreads();
            if (threadIdx.x < SINK_BK) {
                const int j = kv0 + threadIdx.x;
                int page = -1;
                if (j < r_end) {
                    const int b = j / page_size;
                    page = b < table_width ? table[b] : -1;
                    if (page >= n_pages) { atomicOr(status, 8); page = -1; }
                }
                page_s[threadIdx.x] = page;
            }
            __syncthreads();
            if (vec) {
                const int vpr = wrow / N;
                for (int idx = threadIdx.x; idx < SINK_BK * vpr; idx += blockDim.x) {
                    const int j = idx / vpr, c = (idx % vpr) * N;
                    const int page = page_s[j];
                    float f[N];
                    if (page >= 0) {
                        Vec16<T> v;
                        v.load(kv_pool + (((size_t)page * nkv + kh) * page_size + (kv0 + j) % page_size) * wrow + c);
                        v.unpack(f);
                    } else {
#pragma unroll
                        for (int k = 0; k < N; k++) f[k] = 0.f;
                    }
                    float* dst = c < dk ? k_s + j * dkp + c : v_s + j * dvp + (c - dk);
#pragma unroll
                    for (int k = 0; k < N; k++) dst[k] = f[k];
                }
            } else {
                for (int idx = threadIdx.x; idx < SINK_BK * wrow; idx += blockDim.x) {
                    const int j = idx / wrow, c = idx % wrow;
                    const int page = page_s[j];
                    const float f = page >= 0 ? to_f32(kv_pool[(((size_t)page * nkv + kh) * page_size + (kv0 + j) % page_size) * wrow + c]) : 0.f;
                    if (c < dk) k_s[j * dkp + c] = f; else v_s[j * dvp + (c - dk)] = f;
                }
            }
            __syncthreads();
            if (!active) continue;
            const int j = kv0 + lane;
            const bool visible = j < r_end && j <= pos && (window <= 0 || pos - j < window || j < keep_first);
            if (!__any_sync(0xffffffffu, visible)) continue;
            float s = 0.f;
            {
                const float* kr = k_s + lane * dkp;
                const float* qr = q_s + warp * dk;
                if (dk % 4 == 0) {
                    for (int c = 0; c < dk; c += 4) {
                        const float4 a = *reinterpret_cast<const float4*>(qr + c), b = *reinterpret_cast<const float4*>(kr + c);
                        s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
                    }
                } else {
                    for (int c = 0; c < dk; c++) s = fmaf(qr[c], kr[c], s);
                }
            }
            s *= scale;
            if (cap > 0.f) s = cap * tanhf(s * inv_cap);
            s = visible ? s : -CUDART_INF_F;
            const float m_new = fmaxf(m, warp_max(s));
            const float p = visible ? expf(s - m_new) : 0.f;
            const float corr = expf(m - m_new);
            l = l * corr + warp_sum(p);
            m = m_new;
#pragma unroll
            for (int k = 0; k < SINK_MAX_D / 32; k++) acc[k] *= corr;
            for (int jj = 0; jj < SINK_BK; jj++) {
                const float pj = __shfl_sync(0xffffffffu, p, jj);
                if (pj == 0.f) continue;
                const float* vr = v_s + jj * dvp;
#pragma unroll
                for (int k = 0; k < SINK_MAX_D / 32; k++)
                    if (k * 32 + lane < dv) acc[k] = fmaf(pj, vr[k * 32 + lane], acc[k]);
            }
        }
    }
    if (!active) return;
    if (first_split && sinks) {
        // the sink: one more logit in the denominator, no value
        const float s = sinks[head];
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);
        l = l * corr + expf(s - m_new);
        m = m_new;
#pragma unroll
        for (int k = 0; k < SINK_MAX_D / 32; k++) acc[k] *= corr;
    }
    if (w.part_slot < 0) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + ((size_t)(w.q_token0 + tq) * nh + head) * dv;
#pragma unroll
        for (int k = 0; k < SINK_MAX_D / 32; k++)
            if (k * 32 + lane < dv) o[k * 32 + lane] = from_f32<T>(acc[k] * inv);
    } else {
        const size_t pr = (size_t)(w.part_slot + tq) * nh + head;
        float* o = part_o + pr * dv;
#pragma unroll
        for (int k = 0; k < SINK_MAX_D / 32; k++)
            if (k * 32 + lane < dv) o[k * 32 + lane] = acc[k];
        if (lane == 0) { part_ml[pr * 2] = m; part_ml[pr * 2 + 1] = l; }
    }
}

PLLM_EXPORT int pllm_attention_sink(int dtype, const void* q, const void* kv_pool, const int* block_tables, const int* work,
                                    const int* n_work_ptr, int max_work, void* out, float* part_o, float* part_ml,
                                    const float* sinks, int nh, int nkv, int dk, int dv, int page_size, int n_pages, int table_width,
                                    int window, int keep_first, float scale, float cap, int* status, cudaStream_t stream) {
    if (max_work <= 0) return PLLM_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0 || window < 0 || keep_first < 0) return PLLM_ERR_SIZE;
    if (dk <= 0 || dv <= 0) return PLLM_ERR_SIZE;
    if (dk > SINK_MAX_D || dv > SINK_MAX_D) return PLLM_ERR_LIMIT;
    const int group = nh / nkv;
    const int heads_per_cta = group < SINK_MAX_ROWS ? group : SINK_MAX_ROWS;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    // (rows of k_s and v_s start on 16-byte boundaries when dk and dv are multiples of 4; otherwise only scalar reads are made)
    const size_t smem = ((size_t)SINK_MAX_ROWS * dk + (size_t)SINK_BK * (dk + 4) + (size_t)SINK_BK * (dv + 4)) * sizeof(float);
    PLLM_DISPATCH_DTYPE(dtype, {
        cudaFuncSetAttribute(attention_sink_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        dim3 grid(max_work, nkv * gparts);
        launch_chained(attention_sink_kernel<T>, grid, dim3(SINK_MAX_ROWS * 32), smem, stream, (const T*)q, (const T*)kv_pool,
                       block_tables, (const SinkWork*)work, n_work_ptr, (T*)out, part_o, part_ml, sinks, nh, nkv, dk, dv, page_size,
                       n_pages, table_width, window, keep_first, scale, cap, heads_per_cta, status);
    });
    return launch_status();
}

// The most query tokens one work item may hold for a given group size.
PLLM_EXPORT int pllm_attention_sink_tile_tokens(int nh, int nkv) {
    const int group = nh / nkv;
    const int heads_per_cta = group < SINK_MAX_ROWS ? group : SINK_MAX_ROWS;
    return SINK_MAX_ROWS / heads_per_cta;
}

PLLM_TRACE_EXPORT(attention_sink)

// Latent attention: what lies between its down-projections and its attention.
//
// A token's down-projection gives [ q latent (q_rank) | kv latent (kv_rank) ] in one row.  Both are
// RMS-normed (float statistic, gain multiply in float, one rounding); the q latent goes on to the
// up-projection, the kv latent is the ONLY thing the layer caches: one row of kv_rank values a
// token, written to the paged row pool [pages * page_size, kv_rank] at the token's slot.
#include "common.cuh"

enum : int { KID_LATENT = 50 };

template <typename T>
__global__ void __launch_bounds__(256) latent_norm_write_kernel(const T* qa, const float* __restrict__ q_gain,
                                                                const float* __restrict__ kv_gain, float eps, T* __restrict__ cq,
                                                                T* pool, const int* __restrict__ slots, int q_rank, int kv_rank,
                                                                long long pool_rows, int* status) {
    __shared__ float scratch[2][8];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int slot = (pool && slots) ? slots[t] : -1;
    pdl_wait(KID_LATENT);
    constexpr int N = Vec16<T>::N;
    const int total = q_rank + kv_rank;
    const T* row = qa + (size_t)t * total;
    const bool vec = q_rank % N == 0 && kv_rank % N == 0;      // every vector lies in one of the two parts, rows start on 16 bytes
    // a thread's share of the row stays in registers between the statistic and the scaling where it is a vector or two
    float f[2][N];
    float sq = 0.f, sk = 0.f;
    if (vec) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int c = (threadIdx.x + j * blockDim.x) * N;
            if (c < total) {
                Vec16<T> v; v.load(row + c); v.unpack(f[j]);
                float ss = 0.f;
#pragma unroll
                for (int k = 0; k < N; k++) ss += f[j][k] * f[j][k];
                if (c < q_rank) sq += ss; else sk += ss;
            }
        }
        for (int c = (threadIdx.x + 2 * blockDim.x) * N; c < total; c += blockDim.x * N) {      // (rows wider than two vectors a thread)
            Vec16<T> v; v.load(row + c);
            float g[N]; v.unpack(g);
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < N; k++) ss += g[k] * g[k];
            if (c < q_rank) sq += ss; else sk += ss;
        }
    } else {
        for (int c = threadIdx.x; c < total; c += blockDim.x) { const float v = to_f32(row[c]); if (c < q_rank) sq += v * v; else sk += v * v; }
    }
    sq = warp_sum(sq); sk = warp_sum(sk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    if (lane == 0) { scratch[0][warp] = sq; scratch[1][warp] = sk; }
    __syncthreads();
    sq = 0.f; sk = 0.f;
    for (int w = 0; w < warps; w++) { sq += scratch[0][w]; sk += scratch[1][w]; }
    const float iq = 1.0f / sqrtf(sq / (float)q_rank + eps), ik = 1.0f / sqrtf(sk / (float)kv_rank + eps);
    T* cqr = cq + (size_t)t * q_rank;
    const bool writes = slot >= 0 && slot < pool_rows;
    if (slot >= pool_rows && threadIdx.x == 0) atomicOr(status, 2);      // (a negative slot: padding of a captured step, or a run that reads another run's cache)
    T* dst = writes ? pool + (size_t)slot * kv_rank : nullptr;
    if (vec) {
        for (int j = 0, c = threadIdx.x * N; c < total; j++, c += blockDim.x * N) {
            float g[N];
            if (j < 2) {
#pragma unroll
                for (int k = 0; k < N; k++) g[k] = f[j][k];
            } else { Vec16<T> v; v.load(row + c); v.unpack(g); }
            const bool isq = c < q_rank;
            const float* gain = isq ? q_gain + c : kv_gain + (c - q_rank);
            const float inv = isq ? iq : ik;
#pragma unroll
            for (int k = 0; k < N; k++) g[k] = g[k] * inv * gain[k];
            Vec16<T> o; o.pack(g);
            if (isq) o.store(cqr + c);
            else if (dst) o.store(dst + (c - q_rank));
        }
        return;
    }
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) cqr[c] = from_f32<T>(to_f32(row[c]) * iq * q_gain[c]);
    if (!dst) return;
    for (int c = threadIdx.x; c < kv_rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32(row[q_rank + c]) * ik * kv_gain[c]);
}

PLLM_EXPORT int pllm_latent_norm_write(int dtype, const void* qa, const float* q_gain, const float* kv_gain, float eps, void* cq,
                                       void* pool, const int* slots, int n_tokens, int q_rank, int kv_rank, long long pool_rows,
                                       int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (q_rank <= 0 || kv_rank <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int threads = min(256, max(32, ((q_rank + kv_rank) / Vec16<T>::N + 31) / 32 * 32));
        launch_chained(latent_norm_write_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, (const T*)qa, q_gain, kv_gain, eps,
                       (T*)cq, (T*)pool, slots, q_rank, kv_rank, pool_rows, status);
    });
    return launch_status();
}

// ---- attention over the cached latent rows, any sizes, on the CUDA cores ---------------------------------
// Every head of a token attends over the same rows c(j) of its request, and the rows are keys and values
// at once: score = scale * q~ . c(j), output = sum_j p_j c(j) (both kv_rank wide).  Work items, splits of
// long key ranges and their partial results are those of the grouped-query kernels
// (attention_generic.cu, kernels/attention_plan.py), with every head in the one group:
//   item = {seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split}
// One CTA per (item, part of the heads); a warp owns a row (token x head), the softmax runs online over
// tiles of 32 rows of c, and a tile is staged in shared memory once for scores and sums alike.
// The kernel of the float32 engine and of bfloat16 shapes the tensor-core kernel does not take.
#define LAT_BK 32
#define LAT_ROWS 16
#define LAT_MAX_R 1024

struct LatWork { int seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split; };

template <typename T, int KMAX>      // KMAX * 32 >= kv_rank
__global__ void __launch_bounds__(LAT_ROWS * 32) latent_attention_generic_kernel(
    const T* q,                       // [tokens, heads, R]   (just written: no __restrict__)
    const T* pool,                    // [pages * page_size, R]
    const int* __restrict__ block_tables, const LatWork* __restrict__ work, const int* __restrict__ n_work_ptr,
    T* __restrict__ out,              // [tokens, heads, R]
    float* __restrict__ part_o, float* __restrict__ part_ml,
    int heads, int R, int page_size, int n_pages, int table_width, float scale, int heads_per_cta, int* status) {
    pdl_launch_dependents();
    pdl_wait(KID_LATENT);
    if ((int)blockIdx.x >= *n_work_ptr) return;
    const LatWork w = work[blockIdx.x];
    const int head0 = blockIdx.y * heads_per_cta;
    const int n_heads = min(heads_per_cta, heads - head0);
    const int rows = w.q_count * n_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int R4 = (R + 3) & ~3;      // rows in shared memory are whole float4s, zero beyond R
    const int Rp = R4 + 4;            // padded: conflict-free float4 reads across rows

    extern __shared__ float smem[];
    float* q_s = smem;                         // [LAT_ROWS][R4]
    float* c_s = q_s + LAT_ROWS * R4;          // [LAT_BK][Rp]
    __shared__ int page_s[LAT_BK];

    const bool active = warp < rows;
    const int tq = active ? warp / n_heads : 0;
    const int head = active ? head0 + warp % n_heads : head0;
    const int pos = w.q_pos0 + tq;
    if (active) {
        const T* qr = q + ((size_t)(w.q_token0 + tq) * heads + head) * R;
        for (int e = lane; e < R4; e += 32) q_s[warp * R4 + e] = e < R ? to_f32(qr[e]) * scale : 0.f;
    }
    const int lo = w.kv_begin;
    const int hi = min(w.kv_end, pos + 1);

    float m = -CUDART_INF_F, l = 0.f;
    float acc[KMAX];
#pragma unroll
    for (int k = 0; k < KMAX; k++) acc[k] = 0.f;

    constexpr int N = Vec16<T>::N;
    const bool vec = R % N == 0;
    const int* table = block_tables + (size_t)w.seg * table_width;

    for (int kv0 = w.kv_begin; kv0 < w.kv_end; kv0 += LAT_BK) {
        __syncthreads();
        if (threadIdx.x < LAT_BK) {
            const int j = kv0 + threadIdx.x;
            int page = -1;
            if (j < w.kv_end) {
                const int b = j / page_size;
                page = b < table_width ? table[b] : -1;
                if (page >= n_pages) { atomicOr(status, 8); page = -1; }
            }
            page_s[threadIdx.x] = page;
        }
        __syncthreads();
        if (vec) {
            const int vec_per_row = R / N;
            for (int idx = threadIdx.x; idx < LAT_BK * vec_per_row; idx += blockDim.x) {
                const int j = idx / vec_per_row, c = (idx % vec_per_row) * N;
                const int page = page_s[j];
                float f[N];
                if (page >= 0) {
                    Vec16<T> v; v.load(pool + ((size_t)page * page_size + (kv0 + j) % page_size) * R + c);
                    v.unpack(f);
                } else {
#pragma unroll
                    for (int k = 0; k < N; k++) f[k] = 0.f;
                }
#pragma unroll
                for (int k = 0; k < N; k++) c_s[j * Rp + c + k] = f[k];
            }
            if (R4 != R)
                for (int idx = threadIdx.x; idx < LAT_BK * (R4 - R); idx += blockDim.x) c_s[(idx / (R4 - R)) * Rp + R + idx % (R4 - R)] = 0.f;
        } else {
            for (int idx = threadIdx.x; idx < LAT_BK * R4; idx += blockDim.x) {
                const int j = idx / R4, c = idx % R4;
                const int page = page_s[j];
                c_s[j * Rp + c] = (page >= 0 && c < R) ? to_f32(pool[((size_t)page * page_size + (kv0 + j) % page_size) * R + c]) : 0.f;
            }
        }
        __syncthreads();
        if (!active) continue;
        const int j = kv0 + lane;
        const bool visible = j >= lo && j < hi;
        if (!__any_sync(0xffffffffu, visible)) continue;
        float s = 0.f;
        {
            const float4* cr = reinterpret_cast<const float4*>(c_s + lane * Rp);
            const float4* qr = reinterpret_cast<const float4*>(q_s + warp * R4);
            for (int c = 0; c < R4 / 4; c++) {
                const float4 a = qr[c], b = cr[c];
                s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
            }
        }
        s = visible ? s : -CUDART_INF_F;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = visible ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int k = 0; k < KMAX; k++) acc[k] *= corr;
        for (int jj = 0; jj < LAT_BK; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            if (pj == 0.f) continue;
            const float* vr = c_s + jj * Rp;
#pragma unroll
            for (int k = 0; k < KMAX; k++)
                if (k * 32 + lane < R) acc[k] = fmaf(pj, vr[k * 32 + lane], acc[k]);
        }
    }
    if (!active) return;
    if (w.part_slot < 0) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + ((size_t)(w.q_token0 + tq) * heads + head) * R;
#pragma unroll
        for (int k = 0; k < KMAX; k++)
            if (k * 32 + lane < R) o[k * 32 + lane] = from_f32<T>(acc[k] * inv);
    } else {
        const size_t pr = (size_t)(w.part_slot + tq) * heads + head;
        float* o = part_o + pr * R;
#pragma unroll
        for (int k = 0; k < KMAX; k++)
            if (k * 32 + lane < R) o[k * 32 + lane] = acc[k];
        if (lane == 0) { part_ml[pr * 2] = m; part_ml[pr * 2 + 1] = l; }
    }
}

static inline int lat_heads_per_cta(int heads) { return heads < LAT_ROWS ? heads : LAT_ROWS; }

PLLM_EXPORT int pllm_latent_attention_generic_tile_tokens(int heads) { return LAT_ROWS / lat_heads_per_cta(heads); }
PLLM_EXPORT int pllm_latent_attention_generic_ctas_per_item(int heads) {
    return (heads + lat_heads_per_cta(heads) - 1) / lat_heads_per_cta(heads);
}

PLLM_EXPORT int pllm_latent_attention_generic(int dtype, const void* q, const void* pool, const int* block_tables, const int* work,
                                              const int* n_work_ptr, int max_work, void* out, float* part_o, float* part_ml,
                                              int heads, int R, int page_size, int n_pages, int table_width, float scale,
                                              int* status, cudaStream_t stream) {
    if (max_work <= 0) return PLLM_OK;
    if (heads <= 0 || R <= 0 || page_size <= 0) return PLLM_ERR_SIZE;
    if (R > LAT_MAX_R) return PLLM_ERR_LIMIT;
    const int hpc = lat_heads_per_cta(heads);
    const int R4 = (R + 3) & ~3;
    const size_t smem = ((size_t)LAT_ROWS * R4 + (size_t)LAT_BK * (R4 + 4)) * sizeof(float);
    dim3 grid(max_work, (heads + hpc - 1) / hpc);
#define LAT_LAUNCH(KMAX)                                                                                                  \
    do {                                                                                                                  \
        cudaFuncSetAttribute(latent_attention_generic_kernel<T, KMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_chained(latent_attention_generic_kernel<T, KMAX>, grid, dim3(LAT_ROWS * 32), smem, stream, (const T*)q,    \
                       (const T*)pool, block_tables, (const LatWork*)work, n_work_ptr, (T*)out, part_o, part_ml, heads, R, \
                       page_size, n_pages, table_width, scale, hpc, status);                                              \
    } while (0)
    PLLM_DISPATCH_DTYPE(dtype, {
        if (R <= 128) LAT_LAUNCH(4);
        else if (R <= 256) LAT_LAUNCH(8);
        else if (R <= 512) LAT_LAUNCH(16);
        else LAT_LAUNCH(32);
    });
#undef LAT_LAUNCH
    return launch_status();
}

PLLM_TRACE_EXPORT(latent)

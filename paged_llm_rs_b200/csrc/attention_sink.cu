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
//                       Float arithmetic on the CUDA cores, for any sizes: the true 32-bit path.
//   attention_sink_mma  the same on the tensor cores for bfloat16 and key / value sizes of 32, 64 or 128.
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

// ---- the same attention on the tensor cores (bfloat16) ------------------------------------------------------------
// One CTA of four warps per (item, kv head, part of the group) holds up to 64 query rows (token x head of the group,
// ordered as above), 16 a warp.  Keys and values come in tiles of 64 cached tokens, copied as they lie in the pages
// (cp.async, 16 bytes a thread; rows past the range or in pages given back are zero-filled) into padded rows of shared
// memory; S = Q K^T and O += P V are mma.sync m16n8k16 products with float accumulators, the operands fetched with
// ldmatrix (V transposed on the way); scale, cap, mask and the running softmax act on the accumulator registers.  A warp
// skips tiles none of its rows can see.  An item of 16 rows or fewer (decoded tokens) is shared out the other way: every
// warp holds the same rows and takes 16 keys of each tile, and the four partial results meet in shared memory at the end.
// Key and value sizes are template parameters (32, 64 or 128 each).
#define SMMA_BK 64
#define SMMA_ROWS 64
#define SMMA_PAD 8

__device__ __forceinline__ uint32_t sink_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void sink_cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void sink_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
}
__device__ __forceinline__ void sink_ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sink_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void sink_mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t sink_pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int DK, int DV>
__global__ void __launch_bounds__(128, (DK + DV <= 192) ? 4 : 3) attention_sink_mma_kernel(const bf16* q, const bf16* kv_pool, const int* __restrict__ block_tables,
                                                                 const SinkWork* __restrict__ work, const int* __restrict__ n_work_ptr,
                                                                 bf16* __restrict__ out, float* __restrict__ part_o,
                                                                 float* __restrict__ part_ml, const float* __restrict__ sinks, int nh,
                                                                 int nkv, int page_size, int n_pages, int table_width, int window,
                                                                 int keep_first, float scale, float cap, int heads_per_cta, int* status) {
    constexpr int QS = DK + SMMA_PAD, KS = DK + SMMA_PAD, VS = DV + SMMA_PAD;      // row strides in elements
    extern __shared__ __align__(16) unsigned char sink_smem[];
    bf16* q_s = reinterpret_cast<bf16*>(sink_smem);            // [SMMA_ROWS][QS]
    bf16* k_s = q_s;                                           // the tiles' place: the queries' own, once they are in registers
    constexpr int TILE = SMMA_BK * (KS + VS);                  // a tile's keys [SMMA_BK][KS], then its values [SMMA_BK][VS]; two tiles
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
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const bool first_split = (w.split & 0xffff) == 0;
    const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
    constexpr int WROW = DK + DV;

    // the queries of the CTA's rows into shared memory (rows past the item's are zeros)
    for (int idx = threadIdx.x; idx < SMMA_ROWS * (DK / 8); idx += blockDim.x) {
        const int r = idx / (DK / 8), c = (idx % (DK / 8)) * 8;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(q + ((size_t)(w.q_token0 + r / n_heads) * nh + head0 + r % n_heads) * DK + c);
        *reinterpret_cast<uint4*>(q_s + r * QS + c) = v;
    }
    __syncthreads();
    const bool ksplit = rows <= 16;                  // the warps share the keys of a tile, not the rows
    const int row_base = ksplit ? 0 : warp * 16;
    uint32_t qf[DK / 16][4];
#pragma unroll
    for (int kk = 0; kk < DK / 16; kk++)
        sink_ldmatrix_x4(qf[kk], sink_smem_u32(q_s + (row_base + (lane & 7) + ((lane >> 3) & 1) * 8) * QS + kk * 16 + (lane >> 4) * 8));

    __syncthreads();                                 // every warp has its query fragments: the tiles may overwrite them
    // this thread's two rows: r0 = row_base + g and r0 + 8
    const int r0 = row_base + g, r1 = r0 + 8;
    const int pos0 = w.q_pos0 + (r0 < rows ? r0 / n_heads : 0), pos1 = w.q_pos0 + (r1 < rows ? r1 / n_heads : 0);
    const bool live0 = r0 < rows, live1 = r1 < rows;
    // positions of the warp's rows, for skipping tiles: rows warp*16 .. warp*16+15 that exist
    const int wr_lo = row_base, wr_hi = min(rows, row_base + 16) - 1;
    const bool warp_live = wr_lo < rows;
    const int wpos_lo = w.q_pos0 + wr_lo / n_heads, wpos_hi = w.q_pos0 + (warp_live ? wr_hi / n_heads : 0);

    float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.f, l1 = 0.f;
    float o[DV / 8][4];
#pragma unroll
    for (int j = 0; j < DV / 8; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    const int* table = block_tables + (size_t)w.seg * table_width;

    // The tiles of the item, in order: those of the kept first tokens before its range (first split only), then its range.
    const int r0_end = first_split && window > 0 ? min(keep_first, w.kv_begin) : 0;
    const int n0 = (r0_end + SMMA_BK - 1) / SMMA_BK, n_tiles = n0 + (max(w.kv_end - w.kv_begin, 0) + SMMA_BK - 1) / SMMA_BK;
    // Tile i + 1 is on its way (cp.async into the other half of the tiles' place) while tile i is multiplied; a row's
    // page is looked up by the thread that copies it, a tile ahead, so no lookup stands between a tile and its copy.
    auto issue = [&](int i) {
        const int kv0 = i < n0 ? i * SMMA_BK : w.kv_begin + (i - n0) * SMMA_BK, r_end = i < n0 ? r0_end : w.kv_end;
        bf16* kb = k_s + (i & 1) * TILE, * vb = kb + SMMA_BK * KS;
        // four threads a row: the row's page is looked up once, then each copies every fourth 16-byte piece of it
        constexpr int CPR = WROW / 8;
#pragma unroll
        for (int pass = 0; pass < SMMA_BK / 32; pass++) {
            const int j = pass * 32 + (threadIdx.x >> 2), q4 = threadIdx.x & 3;
            int page = -1;
            if (kv0 + j < r_end) {
                const int b = (kv0 + j) / page_size;
                page = b < table_width ? __ldg(table + b) : -1;
                if (page >= n_pages) { atomicOr(status, 8); page = -1; }
            }
            const bf16* src = kv_pool + (((size_t)max(page, 0) * nkv + kh) * page_size + (kv0 + j) % page_size) * WROW;
            bf16* kd = kb + j * KS;
            bf16* vd = vb + j * VS - DK;
#pragma unroll
            for (int k = 0; k < CPR / 4; k++) {
                const int c = (q4 + 4 * k) * 8;
                sink_cp_async16(sink_smem_u32(c < DK ? kd + c : vd + c), src + c, page >= 0);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    if (n_tiles > 0) issue(0);
    for (int i = 0; i < n_tiles; i++) {
        const int kv0 = i < n0 ? i * SMMA_BK : w.kv_begin + (i - n0) * SMMA_BK, r_end = i < n0 ? r0_end : w.kv_end;
        const bf16* k_t = k_s + (i & 1) * TILE;
        const bf16* v_t = k_t + SMMA_BK * KS;
        if (i + 1 < n_tiles) {
            issue(i + 1);
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        __syncthreads();                     // tile i has landed for every thread
        {
            // can any row of this warp see any key of (its share of) the tile?
            const int t_lo = ksplit ? kv0 + warp * 16 : kv0;
            const int t_hi = min(ksplit ? t_lo + 16 : kv0 + SMMA_BK, r_end) - 1;
            bool any = warp_live && t_lo <= wpos_hi && t_lo < r_end;
            if (any && window > 0) any = t_hi > wpos_lo - window || t_lo < keep_first;
            if (any) {
                float sc[SMMA_BK / 8][4];
#pragma unroll
                for (int j = 0; j < SMMA_BK / 8; j++) { sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < DK / 16; kk++) {
#pragma unroll
                    for (int j = 0; j < SMMA_BK / 8; j += 2) {
                        if (ksplit && j != 2 * warp) continue;
                        uint32_t b[4];
                        sink_ldmatrix_x4(b, sink_smem_u32(k_t + (j * 8 + (lane & 7) + (lane >> 4) * 8) * KS + kk * 16 + ((lane >> 3) & 1) * 8));
                        sink_mma_bf16(sc[j], qf[kk], b[0], b[1]);
                        sink_mma_bf16(sc[j + 1], qf[kk], b[2], b[3]);
                    }
                }
                // scale, cap, mask; the tile's row maxima
                float tm0 = -CUDART_INF_F, tm1 = -CUDART_INF_F;
#pragma unroll
                for (int j = 0; j < SMMA_BK / 8; j++) {
                    if (ksplit && (j >> 1) != warp) continue;          // (another warp's keys: left out of everything below)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int key = kv0 + j * 8 + t4 * 2 + (e & 1);
                        const int pos = e < 2 ? pos0 : pos1;
                        const bool live = e < 2 ? live0 : live1;
                        const bool seen = live && key < r_end && key <= pos && (window <= 0 || pos - key < window || key < keep_first);
                        float v = sc[j][e] * scale;
                        // tanh(x) = 1 - 2 / (exp(2x) + 1) with the fast exponential and division: its absolute error (1e-7) is far
                        // below what the bfloat16 operands leave in the score
                        if (cap > 0.f) v = cap * (1.0f - __fdividef(2.0f, __expf(2.0f * v * inv_cap) + 1.0f));
                        v = seen ? v : -CUDART_INF_F;
                        sc[j][e] = v;
                        if (e < 2) tm0 = fmaxf(tm0, v); else tm1 = fmaxf(tm1, v);
                    }
                }
                tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 1)); tm0 = fmaxf(tm0, __shfl_xor_sync(0xffffffffu, tm0, 2));
                tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 1)); tm1 = fmaxf(tm1, __shfl_xor_sync(0xffffffffu, tm1, 2));
                const float mn0 = fmaxf(m0, tm0), mn1 = fmaxf(m1, tm1);
                const float c0 = mn0 == -CUDART_INF_F ? 1.f : __expf(m0 - mn0), c1 = mn1 == -CUDART_INF_F ? 1.f : __expf(m1 - mn1);
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int j = 0; j < SMMA_BK / 8; j++) {
                    if (ksplit && (j >> 1) != warp) continue;
                    sc[j][0] = mn0 == -CUDART_INF_F ? 0.f : __expf(sc[j][0] - mn0);
                    sc[j][1] = mn0 == -CUDART_INF_F ? 0.f : __expf(sc[j][1] - mn0);
                    sc[j][2] = mn1 == -CUDART_INF_F ? 0.f : __expf(sc[j][2] - mn1);
                    sc[j][3] = mn1 == -CUDART_INF_F ? 0.f : __expf(sc[j][3] - mn1);
                    s0 += sc[j][0] + sc[j][1];
                    s1 += sc[j][2] + sc[j][3];
                }
                s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
                s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
                l0 = l0 * c0 + s0; l1 = l1 * c1 + s1;
                m0 = mn0; m1 = mn1;
#pragma unroll
                for (int j = 0; j < DV / 8; j++) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
                // O += P V
#pragma unroll
                for (int kk = 0; kk < SMMA_BK / 16; kk++) {
                    if (ksplit && kk != warp) continue;
                    uint32_t a[4];
                    a[0] = sink_pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
                    a[1] = sink_pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
                    a[2] = sink_pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
                    a[3] = sink_pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
                    for (int j = 0; j < DV / 8; j += 2) {
                        uint32_t b[4];
                        sink_ldmatrix_x4_trans(b, sink_smem_u32(v_t + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + j * 8 + (lane >> 4) * 8));
                        sink_mma_bf16(o[j], a, b[0], b[1]);
                        sink_mma_bf16(o[j + 1], a, b[2], b[3]);
                    }
                }
            }
        }
        __syncthreads();                     // before the copy of tile i + 2 overwrites this half
    }
    if (ksplit) {
        // the four warps' partial results of the same rows meet: (max, sum, output) a warp and row
        float* comb = reinterpret_cast<float*>(k_s);          // [4 warps][16 rows][DV + 2]
        __syncthreads();                                       // the last tile is no longer read
        {
            float* c0 = comb + ((size_t)warp * 16 + g) * (DV + 2);
            float* c1 = c0 + 8 * (DV + 2);
            if (t4 == 0) { c0[0] = m0; c0[1] = l0; c1[0] = m1; c1[1] = l1; }
#pragma unroll
            for (int j = 0; j < DV / 8; j++) {
                c0[2 + j * 8 + t4 * 2] = o[j][0]; c0[2 + j * 8 + t4 * 2 + 1] = o[j][1];
                c1[2 + j * 8 + t4 * 2] = o[j][2]; c1[2 + j * 8 + t4 * 2 + 1] = o[j][3];
            }
        }
        __syncthreads();
        if (warp != 0) return;
        float M0 = -CUDART_INF_F, M1 = -CUDART_INF_F;
#pragma unroll
        for (int wq = 0; wq < 4; wq++) {
            M0 = fmaxf(M0, comb[((size_t)wq * 16 + g) * (DV + 2)]);
            M1 = fmaxf(M1, comb[((size_t)wq * 16 + g + 8) * (DV + 2)]);
        }
        l0 = l1 = 0.f;
#pragma unroll
        for (int j = 0; j < DV / 8; j++) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
#pragma unroll
        for (int wq = 0; wq < 4; wq++) {                       // always in the order of the warps
            const float* c0 = comb + ((size_t)wq * 16 + g) * (DV + 2);
            const float* c1 = c0 + 8 * (DV + 2);
            const float f0 = c0[0] == -CUDART_INF_F ? 0.f : __expf(c0[0] - M0), f1 = c1[0] == -CUDART_INF_F ? 0.f : __expf(c1[0] - M1);
            l0 += c0[1] * f0; l1 += c1[1] * f1;
#pragma unroll
            for (int j = 0; j < DV / 8; j++) {
                o[j][0] = fmaf(c0[2 + j * 8 + t4 * 2], f0, o[j][0]); o[j][1] = fmaf(c0[2 + j * 8 + t4 * 2 + 1], f0, o[j][1]);
                o[j][2] = fmaf(c1[2 + j * 8 + t4 * 2], f1, o[j][2]); o[j][3] = fmaf(c1[2 + j * 8 + t4 * 2 + 1], f1, o[j][3]);
            }
        }
        m0 = M0; m1 = M1;
    }
    // the sink, then the rows leave
#pragma unroll
    for (int half = 0; half < 2; half++) {
        const int r = half ? r1 : r0;
        if (r >= rows) continue;
        const int tq = r / n_heads, head = head0 + r % n_heads;
        float m = half ? m1 : m0, l = half ? l1 : l0, corr = 1.f;
        if (first_split && sinks) {
            const float s = sinks[head];
            const float mn = fmaxf(m, s);
            corr = m == -CUDART_INF_F ? 0.f : expf(m - mn);
            l = l * corr + expf(s - mn);
            m = mn;
        }
        if (w.part_slot < 0) {
            const float f = corr * (l > 0.f ? 1.0f / l : 0.f);
            bf16* dst = out + ((size_t)(w.q_token0 + tq) * nh + head) * DV;
#pragma unroll
            for (int j = 0; j < DV / 8; j++)
                *reinterpret_cast<uint32_t*>(dst + j * 8 + t4 * 2) = sink_pack_bf16(o[j][2 * half] * f, o[j][2 * half + 1] * f);
        } else {
            const size_t pr = (size_t)(w.part_slot + tq) * nh + head;
            float* dst = part_o + pr * DV;
#pragma unroll
            for (int j = 0; j < DV / 8; j++) { dst[j * 8 + t4 * 2] = o[j][2 * half] * corr; dst[j * 8 + t4 * 2 + 1] = o[j][2 * half + 1] * corr; }
            if (t4 == 0) { part_ml[pr * 2] = m; part_ml[pr * 2 + 1] = l; }
        }
    }
}

static inline bool sink_mma_dims(int dk, int dv) { return (dk == 32 || dk == 64 || dk == 128) && (dv == 32 || dv == 64 || dv == 128); }

// Whether the tensor-core kernel takes this shape (bfloat16 only).
PLLM_EXPORT int pllm_attention_sink_mma_supports(int dtype, int nh, int nkv, int dk, int dv) {
    return dtype == PLLM_BF16 && nh > 0 && nkv > 0 && nh % nkv == 0 && sink_mma_dims(dk, dv);
}

PLLM_EXPORT int pllm_attention_sink_mma_tile_tokens(int nh, int nkv) {
    const int group = nh / nkv;
    const int heads_per_cta = group < SMMA_ROWS ? group : SMMA_ROWS;
    return SMMA_ROWS / heads_per_cta;
}

template <int DK, int DV>
static int launch_sink_mma(const void* q, const void* kv_pool, const int* block_tables, const int* work, const int* n_work_ptr, int max_work,
                           void* out, float* part_o, float* part_ml, const float* sinks, int nh, int nkv, int page_size, int n_pages,
                           int table_width, int window, int keep_first, float scale, float cap, int* status, cudaStream_t stream) {
    const int group = nh / nkv;
    const int heads_per_cta = group < SMMA_ROWS ? group : SMMA_ROWS;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    size_t tiles = 2 * ((size_t)SMMA_BK * (DK + SMMA_PAD) + (size_t)SMMA_BK * (DV + SMMA_PAD)) * sizeof(bf16);
    const size_t meet = (size_t)4 * 16 * (DV + 2) * sizeof(float);      // where the warps of a decoded token's item combine (the tiles' place)
    if (tiles < meet) tiles = meet;
    const size_t queries = (size_t)SMMA_ROWS * (DK + SMMA_PAD) * sizeof(bf16);     // (in registers before the first tile lands on them)
    const size_t smem = tiles > queries ? tiles : queries;
    cudaFuncSetAttribute(attention_sink_mma_kernel<DK, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(attention_sink_mma_kernel<DK, DV>, dim3(max_work, nkv * gparts), dim3(128), smem, stream, (const bf16*)q,
                   (const bf16*)kv_pool, block_tables, (const SinkWork*)work, n_work_ptr, (bf16*)out, part_o, part_ml, sinks, nh, nkv,
                   page_size, n_pages, table_width, window, keep_first, scale, cap, heads_per_cta, status);
    return launch_status();
}

PLLM_EXPORT int pllm_attention_sink_mma(const void* q, const void* kv_pool, const int* block_tables, const int* work,
                                        const int* n_work_ptr, int max_work, void* out, float* part_o, float* part_ml,
                                        const float* sinks, int nh, int nkv, int dk, int dv, int page_size, int n_pages, int table_width,
                                        int window, int keep_first, float scale, float cap, int* status, cudaStream_t stream) {
    if (max_work <= 0) return PLLM_OK;
    if (!pllm_attention_sink_mma_supports(PLLM_BF16, nh, nkv, dk, dv) || page_size <= 0 || window < 0 || keep_first < 0) return PLLM_ERR_SIZE;
    if (((uintptr_t)q | (uintptr_t)kv_pool) & 15) return PLLM_ERR_ALIGN;
#define SINK_MMA_CASE(A, B)                                                                                                     \
    if (dk == A && dv == B)                                                                                                     \
        return launch_sink_mma<A, B>(q, kv_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, sinks, nh, nkv, \
                                     page_size, n_pages, table_width, window, keep_first, scale, cap, status, stream);
    SINK_MMA_CASE(32, 32) SINK_MMA_CASE(32, 64) SINK_MMA_CASE(32, 128)
    SINK_MMA_CASE(64, 32) SINK_MMA_CASE(64, 64) SINK_MMA_CASE(64, 128)
    SINK_MMA_CASE(128, 32) SINK_MMA_CASE(128, 64) SINK_MMA_CASE(128, 128)
#undef SINK_MMA_CASE
    return PLLM_ERR_SIZE;
}

// The most query tokens one work item may hold for a given group size.
PLLM_EXPORT int pllm_attention_sink_tile_tokens(int nh, int nkv) {
    const int group = nh / nkv;
    const int heads_per_cta = group < SINK_MAX_ROWS ? group : SINK_MAX_ROWS;
    return SINK_MAX_ROWS / heads_per_cta;
}

PLLM_TRACE_EXPORT(attention_sink)

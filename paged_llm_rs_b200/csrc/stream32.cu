// A residual stream kept in float32 whatever the compute dtype: the kernels of a decoder whose
// residual sum must not be rounded to bfloat16 between layers.
//
//   embed_scaled32      x[t] = table[token[t]] * scale                      (table in T, x in float)
//   sinusoid_add        x[t, 2i] += sin(p_t * f_i),  x[t, 2i+1] += cos(p_t * f_i)   (angle formed in float)
//   round_rows          h = T(x)                                            (what a sublayer's products read)
//   outnorm_add         x[r] += a[r] / sqrt(mean(a[r]^2) + eps) * gain;  h[r] = T(x[r])
//                       (the norm sits on the sublayer's OUTPUT a, the sum stays in float)
//   rmsnorm_from32      y[i] = T(x[r] / sqrt(mean(x[r]^2) + eps) * gain),  r = rows ? rows[i] : i
//
// All statistics, the gain multiply and the sum are float; each output is rounded once.
#include "common.cuh"

enum : int { KID_STREAM32 = 40 };

template <typename T>
__global__ void embed_scaled32_kernel(const int* __restrict__ tokens, const T* __restrict__ table, float* __restrict__ out,
                                      int hidden, int vocab, float scale, int* status) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(status, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? to_f32(src[i]) * scale : 0.f;
}

PLLM_EXPORT int pllm_embed_scaled32(int dtype, const int* tokens, const void* table, float* out, int n_tokens, int hidden,
                                    int vocab, float scale, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (hidden <= 0 || vocab <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int threads = min(256, max(32, (hidden + 31) / 32 * 32));
        launch_chained(embed_scaled32_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const T*)table, out,
                       hidden, vocab, scale, status);
    });
    return launch_status();
}

// inv_freq holds width / 2 frequencies.  The angle is the float product of the position and the
// frequency; sincosf (the accurate one: this library is not built with fast math) reduces it.
__global__ void sinusoid_add_kernel(float* x, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                    int width) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const int t = blockIdx.x;
    const float p = (float)positions[t];
    float* row = x + (size_t)t * width;
    for (int i = threadIdx.x; i < width / 2; i += blockDim.x) {
        float s, c;
        sincosf(p * inv_freq[i], &s, &c);
        float2 v = *reinterpret_cast<float2*>(row + 2 * i);
        v.x += s; v.y += c;
        *reinterpret_cast<float2*>(row + 2 * i) = v;
    }
}

PLLM_EXPORT int pllm_sinusoid_add(float* x, const int* positions, const float* inv_freq, int n_tokens, int width,
                                  cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (width <= 0 || width % 2) return PLLM_ERR_SIZE;
    const int threads = min(256, max(32, (width / 2 + 31) / 32 * 32));
    launch_chained(sinusoid_add_kernel, dim3(n_tokens), dim3(threads), 0, stream, x, positions, inv_freq, width);
    return launch_status();
}

template <typename T>
__global__ void round_rows_kernel(const float* x, T* __restrict__ h, long long total) {
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
        h[i] = from_f32<T>(x[i]);
}

PLLM_EXPORT int pllm_round_rows(int dtype, const float* x, void* h, long long total, cudaStream_t stream) {
    if (total <= 0) return PLLM_OK;
    PLLM_DISPATCH_DTYPE(dtype, {
        const int blocks = (int)min((long long)sm_count() * 8, (total + 255) / 256);
        launch_chained(round_rows_kernel<T>, dim3(blocks), dim3(256), 0, stream, x, (T*)h, total);
    });
    return launch_status();
}

// One row a team of TEAM lanes x warps of a 256-thread CTA: the row of `a` is read once for the
// statistic and once more (from L1) for the sum.  h may be null (a float32 engine reads x itself).
template <typename T>
__global__ void __launch_bounds__(256) outnorm_add_kernel(float* x, const T* a, const float* __restrict__ gain, T* h,
                                                          int n_rows, int width, float eps, int team) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = (warp % team) * 32 + lane, lanes = team * 32;
    const int rows_per_cta = 8 / team;
    const int r = blockIdx.x * rows_per_cta + warp / team;
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const bool live = r < n_rows;
    const T* ar = a + (size_t)(live ? r : 0) * width;
    float ss = 0.f;
    if (live)
        for (int c = member; c < width; c += lanes) { const float v = to_f32(ar[c]); ss += v * v; }
    ss = warp_sum(ss);
    if (team > 1) {
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        ss = 0.f;
        const int first = warp / team * team;
        for (int w = 0; w < team; w++) ss += part[first + w];
    }
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    float* xr = x + (size_t)r * width;
    T* hr = h ? h + (size_t)r * width : nullptr;
    for (int c = member; c < width; c += lanes) {
        const float v = xr[c] + to_f32(ar[c]) * inv * gain[c];
        xr[c] = v;
        if (hr) hr[c] = from_f32<T>(v);
    }
}

PLLM_EXPORT int pllm_outnorm_add(int dtype, float* x, const void* a, const float* gain, void* h, int n_rows, int width,
                                 float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        int team = 1;
        while (team < 8 && width > team * 32 * 16) team *= 2;      // some sixteen elements a lane before a row gets more warps
        const int rows_per_cta = 8 / team;
        launch_chained(outnorm_add_kernel<T>, dim3((n_rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, stream, x,
                       (const T*)a, gain, (T*)h, n_rows, width, eps, team);
    });
    return launch_status();
}

template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_from32_kernel(const float* x, const float* __restrict__ gain, T* __restrict__ y,
                                                             const int* __restrict__ rows, int n_rows, int width, float eps,
                                                             int team) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = (warp % team) * 32 + lane, lanes = team * 32;
    const int rows_per_cta = 8 / team;
    const int i = blockIdx.x * rows_per_cta + warp / team;
    pdl_launch_dependents();
    pdl_wait(KID_STREAM32);
    const bool live = i < n_rows;
    const size_t r = live ? (rows ? (size_t)rows[i] : (size_t)i) : 0;
    const float* xr = x + r * width;
    float ss = 0.f;
    if (live)
        for (int c = member; c < width; c += lanes) { const float v = xr[c]; ss += v * v; }
    ss = warp_sum(ss);
    if (team > 1) {
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        ss = 0.f;
        const int first = warp / team * team;
        for (int w = 0; w < team; w++) ss += part[first + w];
    }
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    T* yr = y + (size_t)i * width;
    for (int c = member; c < width; c += lanes) yr[c] = from_f32<T>(xr[c] * inv * gain[c]);
}

PLLM_EXPORT int pllm_rmsnorm_from32(int dtype, const float* x, const float* gain, void* y, const int* rows, int n_rows,
                                    int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        int team = 1;
        while (team < 8 && width > team * 32 * 16) team *= 2;
        const int rows_per_cta = 8 / team;
        launch_chained(rmsnorm_from32_kernel<T>, dim3((n_rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, stream, x,
                       gain, (T*)y, rows, n_rows, width, eps, team);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(stream32)

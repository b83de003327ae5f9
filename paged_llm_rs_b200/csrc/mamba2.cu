// The Mamba-2 mixer (a selective state space whose decay is one number a head and token) between its two projections.
//
// The input projection leaves, a token, u = [z: inner | x: inner | B: G*N | C: G*N | dt: heads], inner = heads * P.
// With c = silu(conv(x | B | C) + bias), a causal convolution over each channel's last `taps` inputs (zeros before a
// request's start), and per head h (group g = h / (heads / G)):
//     dt_t = softplus(dt_t + dt_bias_h)            a_t = exp(-exp(A_log_h) * dt_t)
//     S_t  = a_t S_(t-1) + dt_t B_t x_t^T          (S is N x P, float, kept for every request between steps)
//     y_t  = S_t^T C_t + D_h x_t
// then y * silu(z), RMS-normed in `norm_groups` equal parts, times a gain: the output projection's input.
// A request's state slot holds S of every head and each channel's last taps - 1 inputs: [heads * N * P | (taps - 1) * channels]
// floats.  Everything behind the convolution is float; each value that leaves for a product is rounded once.
//
// A step is a list of segments {first token, tokens, tokens before, state slot} on the device; grids are sized by the
// list's capacity and a segment of no tokens does nothing, so a captured step replays for any step that fits.
//
//   mamba2_conv        c for every token of the step (a request's earlier inputs from its state slot)
//   mamba2_scan        the recurrence, token by token in float, tokens fetched a chunk at a time; writes y and the new S,
//                      and moves the convolution's inputs of the step's last tokens into the state slot
//   mamba2_gate_norm   y * silu(z), the grouped norm, the gain
#include "common.cuh"

enum : int { KID_MAMBA2 = 80 };

#define M2_CONV_TOKENS 64      // tokens a CTA of the convolution
#define M2_CHUNK 32            // tokens the scan fetches at a time
#define M2_CHUNK_SMALL 8       // ... where a wide state leaves little shared memory
#define M2_MAX_TAPS 16

struct Segment { int first, count, before, slot; };

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

// grid (segments, channel blocks of 128, token chunks); u: [tokens, u_width] with the channels at u_off.
template <typename T>
__global__ void __launch_bounds__(128) mamba2_conv_kernel(const T* u, int u_width, int u_off, const T* __restrict__ conv_w,
                                                          const T* __restrict__ conv_b, const Segment* __restrict__ segs,
                                                          const float* state, long long state_stride, long long conv_off,
                                                          float* __restrict__ c_out, int channels, int taps) {
    pdl_launch_dependents();
    pdl_wait(KID_MAMBA2);
    const Segment s = segs[blockIdx.x];
    const int t0 = blockIdx.z * M2_CONV_TOKENS;
    if (t0 >= s.count) return;
    const int ch = blockIdx.y * 128 + threadIdx.x;
    if (ch >= channels) return;
    float wt[M2_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < M2_MAX_TAPS; j++) wt[j] = j < taps ? to_f32(conv_w[(size_t)ch * taps + j]) : 0.f;
    const float bias = to_f32(conv_b[ch]);
    const float* st = state + (size_t)s.slot * state_stride + conv_off;       // [taps - 1][channels], oldest first
    const int t1 = min(s.count, t0 + M2_CONV_TOKENS);
    for (int t = t0; t < t1; t++) {
        float acc = bias;
#pragma unroll
        for (int j = 0; j < M2_MAX_TAPS; j++) {
            if (j >= taps) break;
            const int r = t - (taps - 1) + j;              // relative to the segment's first token
            float v;
            if (r >= 0) v = to_f32(u[(size_t)(s.first + r) * u_width + u_off + ch]);
            else v = s.before > 0 ? st[(size_t)(taps - 1 + r) * channels + ch] : 0.f;
            acc = fmaf(wt[j], v, acc);
        }
        c_out[(size_t)(s.first + t) * channels + ch] = silu_f(acc);
    }
}

// grid (segments, heads, slices of P): a CTA holds the columns [p0, p0 + P) of a head's state, P = Pf / slices (few
// segments are cut into more slices, so that a prompt's recurrence runs on more SMs than the model has heads);
// thread (part, e): value entry p0 + e, e = tid % P, state rows n = part, part + parts, ...
// MINB: CTAs an SM the registers are bounded for (three for decoded tokens where a thread holds sixteen state rows: more of
// the state's loads and stores in flight; a prompt's long recurrence runs faster with the registers it likes)
template <typename T, int NPT, int MAXT, int CK, int MINB>
__global__ void __launch_bounds__(MAXT, MINB) mamba2_scan_kernel(const T* u, int u_width, int dt_off, int conv_in_off, const float* c, int channels,
                                   const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                                   const Segment* __restrict__ segs, float* state, long long state_stride, long long conv_off,
                                   float* __restrict__ y, int heads, int groups, int Pf, int P, int N, int taps, int parts) {
    constexpr int chunk = CK;                        // tokens fetched at a time
    extern __shared__ float smem[];
    const int NP = NPT * parts;                      // rows of B and C in shared memory: N, padded with zeros to what the threads hold
    float* x_s = smem;                              // [chunk][P]
    float* b_s = x_s + chunk * P;                // [chunk][NP]
    float* c_s = b_s + chunk * NP;               // [chunk][NP]
    float* dt_s = c_s + chunk * NP;              // [chunk] dt, then [chunk] decay
    float* y_s = dt_s + 2 * chunk;               // [chunk][parts][P]
    pdl_launch_dependents();
    pdl_wait(KID_MAMBA2);
    const Segment s = segs[blockIdx.x];
    if (s.count <= 0) return;
    const int h = blockIdx.y, g = h / (heads / groups), p0 = blockIdx.z * P;
    const int inner = heads * Pf;
    const int e = threadIdx.x % P, part = threadIdx.x / P;
    const bool worker = part < parts;
    float* S = state + (size_t)s.slot * state_stride + (size_t)h * N * Pf + p0;
    float st[NPT];
#pragma unroll
    for (int k = 0; k < NPT; k++) {
        const int n = part + k * parts;
        st[k] = (worker && n < N && s.before > 0) ? S[(size_t)n * Pf + e] : 0.f;
    }
    const float A = -expf(a_log[h]), Dh = d_skip[h], bias = dt_bias[h];
    const bool vec4 = P % 4 == 0 && N % 4 == 0 && Pf % 4 == 0 && channels % 4 == 0 && NP % 4 == 0;
    for (int i = threadIdx.x; i < 2 * chunk * NP; i += blockDim.x) b_s[i] = 0.f;      // (the padding rows stay zero)
    for (int t0 = 0; t0 < s.count; t0 += chunk) {
        const int nt = min(chunk, s.count - t0);
        __syncthreads();
        if (vec4) {
            // rows of whole float4s on 16-byte boundaries: four values a load, a thread's loads in flight together
            const int pv = P / 4, nv = N / 4;
            for (int i = threadIdx.x; i < nt * pv; i += blockDim.x)
                *reinterpret_cast<float4*>(x_s + (i / pv) * P + (i % pv) * 4) =
                    *reinterpret_cast<const float4*>(c + (size_t)(s.first + t0 + i / pv) * channels + h * Pf + p0 + (i % pv) * 4);
#pragma unroll 4
            for (int i = threadIdx.x; i < nt * nv; i += blockDim.x) {
                const float* row = c + (size_t)(s.first + t0 + i / nv) * channels + inner + g * N + (i % nv) * 4;
                const float4 bv = *reinterpret_cast<const float4*>(row), cv = *reinterpret_cast<const float4*>(row + groups * N);
                *reinterpret_cast<float4*>(b_s + (i / nv) * NP + (i % nv) * 4) = bv;
                *reinterpret_cast<float4*>(c_s + (i / nv) * NP + (i % nv) * 4) = cv;
            }
        } else {
            for (int i = threadIdx.x; i < nt * P; i += blockDim.x)
                x_s[i] = c[(size_t)(s.first + t0 + i / P) * channels + h * Pf + p0 + i % P];
            for (int i = threadIdx.x; i < nt * N; i += blockDim.x) {
                const size_t row = (size_t)(s.first + t0 + i / N) * channels;
                b_s[(i / N) * NP + i % N] = c[row + inner + g * N + i % N];
                c_s[(i / N) * NP + i % N] = c[row + inner + groups * N + g * N + i % N];
            }
        }
        if (threadIdx.x < nt) {
            const float dt = softplus_f(to_f32(u[(size_t)(s.first + t0 + threadIdx.x) * u_width + dt_off + h]) + bias);
            dt_s[threadIdx.x] = dt;
            dt_s[chunk + threadIdx.x] = expf(A * dt);
        }
        __syncthreads();
        if (worker) {
            // (rows past N hold zeros in b_s and c_s: their state stays zero and adds nothing, so no row is tested here;
            //  a token's B and C come into registers in one go, ahead of the products that need them)
#pragma unroll 2
            for (int t = 0; t < nt; t++) {
                const float dt = dt_s[t], a = dt_s[chunk + t];
                const float dx = dt * x_s[t * P + e];
                const float* bt = b_s + t * NP + part;
                const float* ct = c_s + t * NP + part;
                float bv[NPT], cv[NPT];
#pragma unroll
                for (int k = 0; k < NPT; k++) { bv[k] = bt[k * parts]; cv[k] = ct[k * parts]; }
                float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
                for (int k = 0; k < NPT; k++) {
                    st[k] = fmaf(a, st[k], dx * bv[k]);
                    if (k & 1) acc1 = fmaf(st[k], cv[k], acc1); else acc0 = fmaf(st[k], cv[k], acc0);
                }
                y_s[(t * parts + part) * P + e] = acc0 + acc1;
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < nt * P; i += blockDim.x) {
            const int t = i / P, ee = i % P;
            float acc = 0.f;
            for (int q = 0; q < parts; q++) acc += y_s[(t * parts + q) * P + ee];     // always in the order of the parts
            y[(size_t)(s.first + t0 + t) * inner + h * Pf + p0 + ee] = acc + Dh * x_s[t * P + ee];
        }
    }
    if (worker) {
#pragma unroll
        for (int k = 0; k < NPT; k++) {
            const int n = part + k * parts;
            if (n < N) S[(size_t)n * Pf + e] = st[k];
        }
    }
    // The convolution's state: the last taps - 1 inputs of this head's channels (x), and of its group's B and C by the
    // group's first head.  The convolution kernel has finished; nobody else touches these channels.
    float* cs = state + (size_t)s.slot * state_stride + conv_off;
    const int hpg = heads / groups;
    const int extra = (h % hpg == 0 && blockIdx.z == 0) ? 2 * N : 0;
    for (int i = threadIdx.x; i < P + extra; i += blockDim.x) {
        int ch;
        if (i < P) ch = h * Pf + p0 + i;
        else if (i < P + N) ch = inner + g * N + (i - P);
        else ch = inner + groups * N + g * N + (i - P - N);
        float keep[M2_MAX_TAPS];
#pragma unroll
        for (int k = 0; k < M2_MAX_TAPS; k++) {
            if (k >= taps - 1) break;
            const int r = s.count - (taps - 1) + k;
            if (r >= 0) keep[k] = to_f32(u[(size_t)(s.first + r) * u_width + conv_in_off + ch]);
            else keep[k] = s.before > 0 ? cs[(size_t)(taps - 1 + r) * channels + ch] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < M2_MAX_TAPS; k++) {
            if (k >= taps - 1) break;
            cs[(size_t)k * channels + ch] = keep[k];
        }
    }
}

// One CTA a token; a norm group is reduced by the whole CTA in turn (groups are few).
template <typename T>
__global__ void __launch_bounds__(256) mamba2_gate_norm_kernel(const float* y, const T* u, int u_width, const float* __restrict__ gain,
                                                               T* __restrict__ out, int inner, int norm_groups, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait(KID_MAMBA2);
    const int t = blockIdx.x;
    const int gw = inner / norm_groups;
    const float* yr = y + (size_t)t * inner;
    const T* zr = u + (size_t)t * u_width;
    T* o = out + (size_t)t * inner;
    for (int g = 0; g < norm_groups; g++) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < gw; i += blockDim.x) {
            const float v = yr[g * gw + i] * silu_f(to_f32(zr[g * gw + i]));
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)gw + eps);
        for (int i = threadIdx.x; i < gw; i += blockDim.x) {
            const float v = yr[g * gw + i] * silu_f(to_f32(zr[g * gw + i]));
            o[g * gw + i] = from_f32<T>(v * inv * gain[g * gw + i]);
        }
    }
}

struct ScanArgs {
    int threads; size_t smem; dim3 grid; cudaStream_t stream; const void* u; int u_width, dt_off, conv_in_off; const float* c; int channels;
    const float *dt_bias, *a_log, *d_skip; const int* segs; float* state; long long state_stride, conv_off; float* y;
    int heads, groups, Pf, P, N, taps, parts;
};

template <typename T, int NPT, int MAXT, int CK, int MINB>
static void launch_scan(const ScanArgs& a) {
    cudaFuncSetAttribute(mamba2_scan_kernel<T, NPT, MAXT, CK, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)a.smem);
    launch_chained(mamba2_scan_kernel<T, NPT, MAXT, CK, MINB>, a.grid, dim3(a.threads), a.smem, a.stream, (const T*)a.u, a.u_width, a.dt_off,
                   a.conv_in_off, a.c, a.channels, a.dt_bias, a.a_log, a.d_skip, (const Segment*)a.segs, a.state, a.state_stride,
                   a.conv_off, a.y, a.heads, a.groups, a.Pf, a.P, a.N, a.taps, a.parts);
}

#define M2_SCAN(NPT_, MAXT_) do { if (chunk == M2_CHUNK) launch_scan<T, NPT_, MAXT_, M2_CHUNK, 1>(a); else launch_scan<T, NPT_, MAXT_, M2_CHUNK_SMALL, ((MAXT_) == 256 && (NPT_) == 16) ? 3 : 1>(a); } while (0)
// u: [tokens, 2 inner + 2 G N + heads] of the compute dtype; conv_w [channels, taps], conv_b [channels] of the same;
// dt_bias, a_log, d_skip, gain float; state [slots, state_stride] float; c_buf [tokens, channels] and y_buf [tokens, inner]
// float scratch; out [tokens, inner] of the compute dtype.  max_segment_tokens bounds a segment's tokens (the step's tokens).
PLLM_EXPORT int pllm_mamba2_mix(int dtype, const void* u, const void* conv_w, const void* conv_b, const float* dt_bias,
                                const float* a_log, const float* d_skip, const float* gain, const int* segs, int n_segs,
                                int max_segment_tokens, float* state, long long state_stride, float* c_buf, float* y_buf, void* out,
                                int n_tokens, int heads, int groups, int P, int N, int taps, int norm_groups, float eps,
                                cudaStream_t stream) {
    if (n_tokens <= 0 || n_segs <= 0) return PLLM_OK;
    if (heads <= 0 || groups <= 0 || heads % groups || P <= 0 || N <= 0 || taps < 1 || norm_groups <= 0) return PLLM_ERR_SIZE;
    const int inner = heads * P, channels = inner + 2 * groups * N;
    if (inner % norm_groups) return PLLM_ERR_SIZE;
    if (taps > M2_MAX_TAPS || P > 1024) return PLLM_ERR_LIMIT;
    const int u_width = 2 * inner + 2 * groups * N + heads;
    const long long conv_off = (long long)heads * N * P;
    if (state_stride < conv_off + (long long)(taps - 1) * channels) return PLLM_ERR_SIZE;
    // Slices of P: a step of few segments (a prompt's portion) is cut so that segments x heads x slices fills the SMs
    // (one CTA an SM, or a few more: two CTAs of a long recurrence on one SM take nearly twice as long), slices of at
    // least 16 columns that divide P.
    int slices = 1;
    while (slices < 8 && (long long)n_segs * heads * slices * 2 <= sm_count() + sm_count() / 8 && P % (2 * slices) == 0 && P / (2 * slices) >= 16) slices *= 2;
    // ... and further while a thread would hold more than 16 state rows: three CTAs an SM instead of two keep more of the
    // state's loads and stores in flight when many requests decode
    while (slices < 8 && P % (2 * slices) == 0 && P / (2 * slices) >= 16 && (P / slices) <= 256 &&
           (N + 256 / (P / slices) - 1) / (256 / (P / slices)) > 16) slices *= 2;
    const int Ps = P / slices;
    // threads of the scan: as many parts of Ps threads as fit 256 (1024 where a thread would hold more than 64 state rows;
    // a thread of 1024 holds 32 at most, for the registers to suffice)
    int threads = 256;
    if (Ps > 256 || (N + (256 / Ps) - 1) / (256 / Ps) > 64) threads = 1024;
    const bool big = threads == 1024;
    int parts = threads / Ps;
    if (parts > N) parts = N;
    const int npt = (N + parts - 1) / parts;
    if (npt > (big ? 32 : 64)) return PLLM_ERR_LIMIT;
    threads = (parts * Ps + 31) / 32 * 32;
    if (threads < M2_CHUNK) threads = M2_CHUNK;
    // (state rows a thread as the kernels are instantiated: the rows of B and C in shared memory are padded to that)
    const int npt_t = big ? (npt <= 8 ? 8 : npt <= 16 ? 16 : 32) : (npt <= 4 ? 4 : npt <= 8 ? 8 : npt <= 16 ? 16 : npt <= 32 ? 32 : 64);
    int chunk = M2_CHUNK;
    auto smem_of = [&](int ck) { return ((size_t)ck * Ps + 2 * (size_t)ck * npt_t * parts + 2 * ck + (size_t)ck * parts * Ps) * sizeof(float); };
    if (smem_of(chunk) > 160 * 1024 || max_segment_tokens <= M2_CHUNK_SMALL) chunk = M2_CHUNK_SMALL;   // (decoded tokens need no more)
    const size_t smem = smem_of(chunk);
    if (smem > 200 * 1024) return PLLM_ERR_LIMIT;
    const int chunks = (max_segment_tokens + M2_CONV_TOKENS - 1) / M2_CONV_TOKENS;
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(mamba2_conv_kernel<T>, dim3(n_segs, (channels + 127) / 128, chunks > 0 ? chunks : 1), dim3(128), 0, stream,
                       (const T*)u, u_width, inner, (const T*)conv_w, (const T*)conv_b, (const Segment*)segs, (const float*)state,
                       state_stride, conv_off, c_buf, channels, taps);
        ScanArgs a{threads, smem, dim3(n_segs, heads, slices), stream, u, u_width, 2 * inner + 2 * groups * N, inner, c_buf, channels, dt_bias,
                   a_log, d_skip, segs, state, state_stride, conv_off, y_buf, heads, groups, P, Ps, N, taps, parts};
        if (big) {
            if (npt_t == 8) M2_SCAN(8, 1024); else if (npt_t == 16) M2_SCAN(16, 1024); else M2_SCAN(32, 1024);
        } else if (npt_t == 4) M2_SCAN(4, 256);
        else if (npt_t == 8) M2_SCAN(8, 256);
        else if (npt_t == 16) M2_SCAN(16, 256);
        else if (npt_t == 32) M2_SCAN(32, 256);
        else M2_SCAN(64, 256);
        launch_chained(mamba2_gate_norm_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (const float*)y_buf, (const T*)u, u_width, gain,
                       (T*)out, inner, norm_groups, eps);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(mamba2)

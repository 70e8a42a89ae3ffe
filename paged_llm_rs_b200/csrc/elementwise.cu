// Embedding gather, RMSNorm (plain, with the residual add fused in, and over
// gathered rows), and the SwiGLU activation.
//
// Formulas follow the reference: embedding is a plain row gather with no scale
// (crates/pagedllm/src/model/mod.rs:323-327); RMSNorm is x / sqrt(mean(x^2) + eps)
// times the gain with the statistic in float (crates/pagedllm/src/model/layers.rs:58-64);
// SwiGLU is silu(gate) * up with the activation on the gate (layers.rs:93-99).
// Here the whole norm, gain multiply included, runs in float and rounds once.
#include "common.cuh"

// Off by default: measured on a B200 with the kernels as they are (each lets its
// dependents in at its first instruction), a decode step of the 0.6B shape was 3 to 6 %
// slower with it (batch 8: 2.26 ms against 2.13 ms): the waiting CTAs of the next
// kernel hold places that the running kernel's later CTAs want.
int pllm_pdl_enabled = 0;

// Switch programmatic dependent launch on (1) or off (0, the default) for every kernel
// of the library; returns the former setting.
// Streaming multiprocessors of the current device (what the kernels size their grids by).
PLLM_EXPORT int pllm_sm_count() { return sm_count(); }

PLLM_EXPORT int pllm_set_pdl(int on) {
    const int was = pllm_pdl_enabled;
    pllm_pdl_enabled = on ? 1 : 0;
    return was;
}

// ---------------------------------------------------------------- embedding
// out[t, :] = table[token[t], :].  A token id outside [0, vocab) writes zeros and
// raises bit 0 of *status.
template <typename T>
__global__ void embed_kernel(const int* __restrict__ tokens, const T* __restrict__ table, T* __restrict__ out,
                             int hidden, int vocab, int* status) {
    pdl_launch_dependents();
    pdl_wait(KID_EMBED);
    const int t = blockIdx.x;
    const int tok = tokens[t];
    const bool ok = tok >= 0 && tok < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(status, 1);
    const T* src = table + (size_t)(ok ? tok : 0) * hidden;
    T* dst = out + (size_t)t * hidden;
    constexpr int N = Vec16<T>::N;
    if (hidden % N == 0) {
        for (int i = threadIdx.x * N; i < hidden; i += blockDim.x * N) {
            Vec16<T> v;
            if (ok) v.load(src + i);
            else { float z[N] = {}; v.pack(z); }
            v.store(dst + i);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? src[i] : from_f32<T>(0.f);
    }
}

PLLM_EXPORT int pllm_embed(int dtype, const int* tokens, const void* table, void* out, int n_tokens, int hidden,
                           int vocab, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    if (hidden <= 0 || vocab <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        int threads = min(256, max(32, (hidden / Vec16<T>::N + 31) / 32 * 32));
        launch_chained(embed_kernel<T>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const T*)table, (T*)out,
                       hidden, vocab, status);
    });
    return launch_status();
}

// ------------------------------------------------------------------ RMSNorm
// Row i of the launch reads source row r = rows ? rows[i] : i.
//   v = x[r] (+ delta[r], rounded to T as the residual stream holds it)
//   if residual_out: residual_out[r] = v         (the fused residual add)
//   y[i] = v / sqrt(mean(v^2) + eps) * gain
// x and residual_out may be the same buffer.
template <typename T>
__global__ void __launch_bounds__(1024) rmsnorm_kernel(const T* x, const T* delta, T* residual_out,   // x, delta: just written, no __restrict__
                               const float* __restrict__ gain, T* __restrict__ y, const int* __restrict__ rows,
                               int width, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int i = blockIdx.x;
    constexpr int N = Vec16<T>::N;
    const bool vec = (width % N == 0);
    // Rows of up to RMS_HELD vectors a thread stay in registers between the two passes; wider rows
    // (and rows that are not whole vectors) are read back.
    constexpr int RMS_HELD = 4;
    const bool held = vec && width <= (int)blockDim.x * N * RMS_HELD;
    // the gain of a thread's first vector (a weight; all of the row when it is at most a vector a thread wide)
    // and the row's number (the step's buffer) are fetched before the wait for the kernel before
    float g0[N];
    {
        const int c = threadIdx.x * N;
#pragma unroll
        for (int k = 0; k < N; k += 4) {
            const float4 q = (held && c < width) ? *reinterpret_cast<const float4*>(gain + c + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            g0[k] = q.x; g0[k + 1] = q.y; g0[k + 2] = q.z; g0[k + 3] = q.w;
        }
    }
    const size_t r = rows ? (size_t)rows[i] : (size_t)i;
    pdl_wait(KID_RMSNORM);
    const T* xr = x + r * width;
    const T* dr = delta ? delta + r * width : nullptr;
    T* rr = residual_out ? residual_out + r * width : nullptr;
    T* yr = y + (size_t)i * width;
    float ss = 0.f;
    if (held) {
        float f[RMS_HELD][N];
#pragma unroll
        for (int j = 0; j < RMS_HELD; j++) {
            const int c = (threadIdx.x + j * blockDim.x) * N;
            if (c >= width) break;
            Vec16<T> v; v.load(xr + c);
            v.unpack(f[j]);
            if (dr) {
                Vec16<T> d; d.load(dr + c);
                float g[N]; d.unpack(g);
#pragma unroll
                for (int k = 0; k < N; k++) f[j][k] = to_f32(from_f32<T>(f[j][k] + g[k]));
                if (rr) { Vec16<T> o; o.pack(f[j]); o.store(rr + c); }
            } else if (rr && rr != xr) {
                v.store(rr + c);
            }
#pragma unroll
            for (int k = 0; k < N; k++) ss += f[j][k] * f[j][k];
        }
        ss = block_sum(ss, scratch);
        const float inv = 1.0f / sqrtf(ss / (float)width + eps);
#pragma unroll
        for (int j = 0; j < RMS_HELD; j++) {
            const int c = (threadIdx.x + j * blockDim.x) * N;
            if (c >= width) break;
            float gg[N];
#pragma unroll
            for (int k = 0; k < N; k += 4) {
                const float4 q = j == 0 ? make_float4(g0[k], g0[k + 1], g0[k + 2], g0[k + 3]) : *reinterpret_cast<const float4*>(gain + c + k);
                gg[k] = q.x; gg[k + 1] = q.y; gg[k + 2] = q.z; gg[k + 3] = q.w;
            }
#pragma unroll
            for (int k = 0; k < N; k++) f[j][k] = f[j][k] * inv * gg[k];
            Vec16<T> o; o.pack(f[j]); o.store(yr + c);
        }
        return;
    }
    if (vec) {
        for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {
            Vec16<T> v; v.load(xr + c);
            float f[N]; v.unpack(f);
            if (dr) {
                Vec16<T> d; d.load(dr + c);
                float g[N]; d.unpack(g);
#pragma unroll
                for (int k = 0; k < N; k++) f[k] = to_f32(from_f32<T>(f[k] + g[k]));
                if (rr) { Vec16<T> o; o.pack(f); o.store(rr + c); }
            } else if (rr && rr != xr) {
                v.store(rr + c);
            }
#pragma unroll
            for (int k = 0; k < N; k++) ss += f[k] * f[k];
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float f = to_f32(xr[c]);
            if (dr) { f = to_f32(from_f32<T>(f + to_f32(dr[c]))); if (rr) rr[c] = from_f32<T>(f); }
            else if (rr && rr != xr) rr[c] = xr[c];
            ss += f * f;
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    // Second pass: the summed row is read back from where it was written, or
    // recomputed from x and delta when nothing was written (gathered rows).
    if (vec) {
        for (int c = threadIdx.x * N; c < width; c += blockDim.x * N) {
            float f[N];
            if (rr) { Vec16<T> v; v.load(rr + c); v.unpack(f); }
            else {
                Vec16<T> v; v.load(xr + c); v.unpack(f);
                if (dr) {
                    Vec16<T> d; d.load(dr + c);
                    float g[N]; d.unpack(g);
#pragma unroll
                    for (int k = 0; k < N; k++) f[k] = to_f32(from_f32<T>(f[k] + g[k]));
                }
            }
#pragma unroll
            for (int k = 0; k < N; k++) f[k] = f[k] * inv * gain[c + k];
            Vec16<T> o; o.pack(f); o.store(yr + c);
        }
    } else {
        for (int c = threadIdx.x; c < width; c += blockDim.x) {
            float f;
            if (rr) f = to_f32(rr[c]);
            else { f = to_f32(xr[c]); if (dr) f = to_f32(from_f32<T>(f + to_f32(dr[c]))); }
            yr[c] = from_f32<T>(f * inv * gain[c]);
        }
    }
}

// The same for many rows (a prompt portion): a row belongs to a team of TEAM warps (1 to 8) of a
// 256-thread CTA, a lane holds up to RMS_TEAM_HELD vectors of it, and the gain is fetched before the
// wait for the kernel before (it is a weight).  With one CTA of `width / 8` threads a row, every
// thread has a single load in flight and the row's sum goes through two CTA barriers; 2048 rows of
// 1024 took 5.2 us in the chain of a 2048-token step that way.
constexpr int RMS_TEAM_HELD = 4;
template <typename T>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const T* x, const T* delta, T* residual_out,   // no __restrict__: see above
                                                            const float* __restrict__ gain, T* __restrict__ y,
                                                            const int* __restrict__ rows, int n_rows, int width, float eps,
                                                            int team) {
    __shared__ float part[8];
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = (warp % team) * 32 + lane, lanes = team * 32;     // this thread's place in its row's team
    const int rows_per_cta = 8 / team;
    const int i = blockIdx.x * rows_per_cta + warp / team;
    pdl_launch_dependents();
    float g[RMS_TEAM_HELD][N];
#pragma unroll
    for (int j = 0; j < RMS_TEAM_HELD; j++) {
        const int c = (member + j * lanes) * N;
#pragma unroll
        for (int k = 0; k < N; k += 4) {
            const float4 q = c < width ? *reinterpret_cast<const float4*>(gain + c + k) : make_float4(0.f, 0.f, 0.f, 0.f);
            g[j][k] = q.x; g[j][k + 1] = q.y; g[j][k + 2] = q.z; g[j][k + 3] = q.w;
        }
    }
    pdl_wait(KID_RMSNORM);
    const bool live = i < n_rows;
    const size_t r = live ? (rows ? (size_t)rows[i] : (size_t)i) : 0;
    const T* xr = x + r * width;
    const T* dr = delta ? delta + r * width : nullptr;
    T* rr = residual_out ? residual_out + r * width : nullptr;
    float f[RMS_TEAM_HELD][N];
    float ss = 0.f;
    if (live) {
        Vec16<T> v[RMS_TEAM_HELD], d[RMS_TEAM_HELD];
#pragma unroll
        for (int j = 0; j < RMS_TEAM_HELD; j++) {
            const int c = (member + j * lanes) * N;
            if (c < width) { v[j].load(xr + c); if (dr) d[j].load(dr + c); }
        }
#pragma unroll
        for (int j = 0; j < RMS_TEAM_HELD; j++) {
            const int c = (member + j * lanes) * N;
            if (c >= width) {
#pragma unroll
                for (int k = 0; k < N; k++) f[j][k] = 0.f;
                continue;
            }
            v[j].unpack(f[j]);
            if (dr) {
                float e[N]; d[j].unpack(e);
#pragma unroll
                for (int k = 0; k < N; k++) f[j][k] = to_f32(from_f32<T>(f[j][k] + e[k]));
                if (rr) { Vec16<T> o; o.pack(f[j]); o.store(rr + c); }
            } else if (rr && rr != xr) {
                v[j].store(rr + c);
            }
#pragma unroll
            for (int k = 0; k < N; k++) ss += f[j][k] * f[j][k];
        }
    }
    ss = warp_sum(ss);
    if (team > 1) {                     // (every warp of the CTA comes here, live or not)
        if (lane == 0) part[warp] = ss;
        __syncthreads();
        ss = 0.f;
        const int first = warp / team * team;
        for (int w = 0; w < team; w++) ss += part[first + w];
    }
    if (!live) return;
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    T* yr = y + (size_t)i * width;
#pragma unroll
    for (int j = 0; j < RMS_TEAM_HELD; j++) {
        const int c = (member + j * lanes) * N;
        if (c >= width) continue;
#pragma unroll
        for (int k = 0; k < N; k++) f[j][k] = f[j][k] * inv * g[j][k];
        Vec16<T> o; o.pack(f[j]); o.store(yr + c);
    }
}

// From how many rows on the team kernel runs (a setter for tuning runs and tests).  Back to back in a captured loop,
// rows of 1024 with the add, microseconds teams / a CTA a row: 512 rows 2.75 / 2.52, 2048: 2.97 / 4.12, 8192: 9.3 / 11.2;
// 2048 rows of 4096: 10.3 / 13.8, of 5120: 15.1 / 25.1.
static int g_rmsnorm_rows_threshold = 1024;
PLLM_EXPORT void pllm_set_rmsnorm_rows_threshold(int n) { g_rmsnorm_rows_threshold = n; }

PLLM_EXPORT int pllm_rmsnorm(int dtype, const void* x, const void* delta, void* residual_out, const float* gain,
                             void* y, const int* rows, int n_rows, int width, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (width <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        if (n_rows >= g_rmsnorm_rows_threshold && width % N == 0 && width <= 8 * 32 * N * RMS_TEAM_HELD) {
            int team = 1;
            while (width > team * 32 * N * RMS_TEAM_HELD) team *= 2;
            const int rows_per_cta = 8 / team;
            launch_chained(rmsnorm_rows_kernel<T>, dim3((n_rows + rows_per_cta - 1) / rows_per_cta), dim3(256), 0, stream,
                           (const T*)x, (const T*)delta, (T*)residual_out, gain, (T*)y, rows, n_rows, width, eps, team);
            return launch_status();
        }
        int threads = min(1024, max(32, (width / Vec16<T>::N + 31) / 32 * 32));
        // A thread that wrote residual_out reads the same addresses back in the
        // second pass (same thread, same columns), so no fence is needed.
        launch_chained(rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), 0, stream, (const T*)x, (const T*)delta,
                       (T*)residual_out, gain, (T*)y, rows, width, eps);
    });
    return launch_status();
}

// ------------------------------------------------------------------- SwiGLU
// in is [n, 2*inter]: the gate in columns [0, inter), up in [inter, 2*inter).
// out[n, inter] = silu(gate) * up, silu(z) = z / (1 + exp(-z)).
template <typename T>
__global__ void swiglu_kernel(const T* in, T* __restrict__ out, int inter, long long total_vec,
                              int vec_per_row) {
    constexpr int N = Vec16<T>::N;
    pdl_launch_dependents();
    pdl_wait(KID_SWIGLU);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total_vec;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / vec_per_row;
        const int c = (int)(idx % vec_per_row) * N;
        const T* g = in + row * 2 * inter + c;
        Vec16<T> vg, vu; vg.load(g); vu.load(g + inter);
        float fg[N], fu[N];
        vg.unpack(fg); vu.unpack(fu);
#pragma unroll
        for (int k = 0; k < N; k++) fg[k] = fg[k] / (1.0f + expf(-fg[k])) * fu[k];
        Vec16<T> o; o.pack(fg); o.store(out + row * inter + c);
    }
}
template <typename T>
__global__ void swiglu_scalar_kernel(const T* in, T* __restrict__ out, int inter, long long total) {
    pdl_launch_dependents();
    pdl_wait(KID_SWIGLU);
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / inter;
        const int c = (int)(idx % inter);
        const float g = to_f32(in[row * 2 * inter + c]), u = to_f32(in[row * 2 * inter + inter + c]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

PLLM_EXPORT int pllm_swiglu(int dtype, const void* in, void* out, int n_rows, int inter, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (inter <= 0) return PLLM_ERR_SIZE;
    PLLM_DISPATCH_DTYPE(dtype, {
        constexpr int N = Vec16<T>::N;
        if (inter % N == 0) {
            long long total = (long long)n_rows * (inter / N);
            int blocks = (int)min((long long)sm_count() * 16, (total + 255) / 256);
            launch_chained(swiglu_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)in, (T*)out, inter, total,
                           inter / N);
        } else {
            long long total = (long long)n_rows * inter;
            int blocks = (int)min((long long)sm_count() * 16, (total + 255) / 256);
            launch_chained(swiglu_scalar_kernel<T>, dim3(blocks), dim3(256), 0, stream, (const T*)in, (T*)out, inter,
                           total);
        }
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(elementwise)

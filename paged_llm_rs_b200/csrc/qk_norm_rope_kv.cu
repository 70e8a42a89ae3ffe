// Fused per-head RMSNorm of q and k, rotary position encoding, and the write of
// k and v into the paged cache.
//
// Order as in the reference (crates/pagedllm/src/model/attention.rs:148-158): the
// norm runs over one head's width with one gain shared by all heads, before the
// rotation; v gets neither; keys are cached after norm and rotation, values raw.
// Rotation pairs dimension i with i + rotary_dim/2 (crates/pagedllm/src/model/rope.rs:96-107):
//   y[i]        = x[i] * cos - x[i + half] * sin
//   y[i + half] = x[i + half] * cos + x[i] * sin
// cos/sin come from a float table [max_positions, rotary_dim/2] whose angles were
// formed in double on the host (rope.rs:39-56).
//
// Cache layout of one layer: [pages, kv_heads, page_size, head_dim]; slot s of the
// request's table means page s / page_size, offset s % page_size.  With `swizzle`
// the 16-byte chunks of a row are stored at chunk index c ^ (offset & 7): the layout
// the tensor-core attention kernels read from shared memory without bank conflicts,
// so that a page can be copied there as it lies.
#include "common.cuh"

template <typename T>
__global__ void qk_norm_rope_kv_kernel(
    const T* qkv,        // [n_tokens, (nh + 2*nkv) * hd]; just written by the projection: no __restrict__
    T* __restrict__ q_out,            // [n_tokens, nh * hd]
    const float* __restrict__ q_gain, // [hd] or null: no q norm
    const float* __restrict__ k_gain, // [hd] or null: no k norm
    float eps,
    const float* __restrict__ cos_t, const float* __restrict__ sin_t,  // [max_pos, rot/2] or null: no rotation
    int rotary_dim, int max_pos,
    const int* __restrict__ positions,  // [n_tokens]
    const int* __restrict__ slots,      // [n_tokens]; < 0: do not write this token
    T* __restrict__ k_pool, T* __restrict__ v_pool,  // null: no cache write at all
    int n_tokens, int nh, int nkv, int hd, int page_size, int n_pages, int swizzle, int* status) {
    extern __shared__ float smem[];  // [warps][hd]
    pdl_launch_dependents();
    pdl_wait(KID_QK);
    const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = nh + 2 * nkv;
    const long long item = (long long)blockIdx.x * warps + warp;
    if (item >= (long long)n_tokens * heads) return;
    const int t = (int)(item / heads), h = (int)(item % heads);
    float* buf = smem + warp * hd;
    const T* src = qkv + (size_t)t * heads * hd + (size_t)h * hd;

    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);

    float ss = 0.f;
    for (int e = lane; e < hd; e += 32) {
        const float f = to_f32(src[e]);
        buf[e] = f;
        ss += f * f;
    }
    if (gain) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
        // The reference rounds the normalised value to the model dtype before the
        // rotation; one rounding at the end is at least as exact.
        for (int e = lane; e < hd; e += 32) buf[e] = buf[e] * inv * gain[e];
    }
    __syncwarp();

    T* dst;
    int xr = 0;  // what a cache row's 16-byte chunks are XOR-ed with (0: stored as they are)
    constexpr int EPC = 16 / (int)sizeof(T);
    if (is_q) {
        dst = q_out + (size_t)t * nh * hd + (size_t)h * hd;
    } else {
        const int slot = slots[t];
        if (!k_pool || slot < 0) return;
        const int page = slot / page_size, off = slot % page_size;
        if (page >= n_pages) { if (lane == 0) atomicOr(status, 2); return; }
        const int kh = is_k ? h - nh : h - nh - nkv;
        dst = (is_k ? k_pool : v_pool) + (((size_t)page * nkv + kh) * page_size + off) * hd;
        if (swizzle) xr = off & 7;
    }
    auto at = [&](int e) { return (((e / EPC) ^ xr) * EPC) + (e % EPC); };

    if ((is_q || is_k) && cos_t) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) { if (lane == 0) atomicOr(status, 4); pos = 0; }
        const int half = rotary_dim >> 1;
        const float* c = cos_t + (size_t)pos * half;
        const float* s = sin_t + (size_t)pos * half;
        for (int i = lane; i < half; i += 32) {
            const float x1 = buf[i], x2 = buf[i + half];
            dst[at(i)] = from_f32<T>(x1 * c[i] - x2 * s[i]);
            dst[at(i + half)] = from_f32<T>(x2 * c[i] + x1 * s[i]);
        }
        for (int e = rotary_dim + lane; e < hd; e += 32) dst[at(e)] = from_f32<T>(buf[e]);
    } else {
        for (int e = lane; e < hd; e += 32) dst[at(e)] = from_f32<T>(buf[e]);
    }
}

// The same, sixteen bytes a lane: LPH lanes share a head (its LPH chunks of 16 bytes), so a
// warp does 32 / LPH heads at once.  The rotation's partner of chunk c is chunk
// c ^ (LPH / 2), one shuffle away; the swizzle is an XOR on the chunk index.  Takes head
// sizes of 8, 16 or 32 chunks that are rotated over their whole width (or not at all).
template <typename T, int LPH>
__global__ void qk_norm_rope_kv_vec_kernel(
    const T* qkv, T* __restrict__ q_out, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    int max_pos, const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ k_pool,
    T* __restrict__ v_pool, int n_tokens, int nh, int nkv, int page_size, int n_pages, int swizzle, int* status) {
    constexpr int N = Vec16<T>::N, HD = LPH * N, HPW = 32 / LPH;
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, sub = lane / LPH, c = lane % LPH;
    const int heads = nh + 2 * nkv;
    const long long total = (long long)n_tokens * heads;
    long long item = ((long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * HPW + sub;
    const bool live = item < total;
    if (!live) item = total - 1;               // idle lanes still take part in the shuffles
    const int t = (int)(item / heads), h = (int)(item % heads);
    const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
    const float* gain = is_q ? q_gain : (is_k ? k_gain : nullptr);
    // What does not come from the kernel before (the token's position and slot out of the step's buffer, the
    // rotation's table, the gain) is fetched before the wait for it: two trips to memory beside its end.
    constexpr int HALF = HD / 2;
    const bool upper = c >= LPH / 2;
    float cs[N], sn[N], gn[N];
    if (cos_t) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) { if (c == 0 && live) atomicOr(status, 4); pos = 0; }
        const size_t o = (size_t)pos * HALF + (upper ? c - LPH / 2 : c) * N;
#pragma unroll
        for (int k = 0; k < N; k++) { cs[k] = cos_t[o + k]; sn[k] = sin_t[o + k]; }
    }
    if (gain) {
#pragma unroll
        for (int k = 0; k < N; k++) gn[k] = gain[c * N + k];
    }
    const int slot = (live && !is_q && k_pool) ? slots[t] : -1;
    pdl_wait(KID_QK);

    Vec16<T> v;
    v.load(qkv + (size_t)t * heads * HD + (size_t)h * HD + c * N);
    float f[N];
    v.unpack(f);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < N; k++) ss += f[k] * f[k];
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (gain) {
        const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int k = 0; k < N; k++) f[k] = f[k] * inv * gn[k];
    }
    if (cos_t) {
#pragma unroll
        for (int k = 0; k < N; k++) {
            const float other = __shfl_xor_sync(0xffffffffu, f[k], LPH / 2);
            if (is_q || is_k) f[k] = upper ? f[k] * cs[k] + other * sn[k] : f[k] * cs[k] - other * sn[k];
        }
    }
    if (!live) return;
    T* dst;
    int xr = 0;
    if (is_q) {
        dst = q_out + (size_t)t * nh * HD + (size_t)h * HD;
    } else {
        if (!k_pool || slot < 0) return;
        const int page = slot / page_size, off = slot % page_size;
        if (page >= n_pages) { if (c == 0) atomicOr(status, 2); return; }
        const int kh = is_k ? h - nh : h - nh - nkv;
        dst = (is_k ? k_pool : v_pool) + (((size_t)page * nkv + kh) * page_size + off) * HD;
        if (swizzle) xr = off & 7;
    }
    v.pack(f);
    v.store(dst + (c ^ xr) * N);
}

// The same for the many tokens of a prompt portion: the four warps of a CTA share one token, each
// taking every fourth run of its heads, 32 / LPH heads at a time, so that the token's rotation
// angles and the two gains are fetched once a warp and not once a head, four heads' loads are in
// flight together, and an SM holds some fifty warps (with a warp a token it held fourteen, and the
// kernel waited on its loads: 15.0 us for the 2048 tokens of the 0.6B shape).
template <typename T, int LPH>
__global__ void __launch_bounds__(128) qk_norm_rope_kv_token_kernel(
    const T* qkv, T* __restrict__ q_out, const float* __restrict__ q_gain,
    const float* __restrict__ k_gain, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
    int max_pos, const int* __restrict__ positions, const int* __restrict__ slots, T* __restrict__ k_pool,
    T* __restrict__ v_pool, int n_tokens, int nh, int nkv, int page_size, int n_pages, int swizzle, int* status) {
    constexpr int N = Vec16<T>::N, HD = LPH * N, HPW = 32 / LPH, UNR = 4;
    pdl_launch_dependents();
    // (position, slot, rotation table and gains do not come from the kernel before: they are fetched before the wait for it)
    const int lane = threadIdx.x & 31, sub = lane / LPH, c = lane % LPH;
    const int t = blockIdx.x, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    if (t >= n_tokens) return;
    const int heads = nh + 2 * nkv;
    float cs[N], sn[N], gq[N], gk[N];
    const bool upper = c >= LPH / 2;
    if (cos_t) {
        int pos = positions[t];
        if (pos < 0 || pos >= max_pos) { if (lane == 0) atomicOr(status, 4); pos = 0; }
        // (N values = 16 or 32 bytes from a multiple of N: vector loads)
        const size_t o = (size_t)pos * (HD / 2) + (upper ? c - LPH / 2 : c) * N;
#pragma unroll
        for (int k = 0; k < N; k += 4) {
            const float4 a = *reinterpret_cast<const float4*>(cos_t + o + k), b = *reinterpret_cast<const float4*>(sin_t + o + k);
            cs[k] = a.x; cs[k + 1] = a.y; cs[k + 2] = a.z; cs[k + 3] = a.w;
            sn[k] = upper ? b.x : -b.x; sn[k + 1] = upper ? b.y : -b.y; sn[k + 2] = upper ? b.z : -b.z; sn[k + 3] = upper ? b.w : -b.w;
        }
    }
#pragma unroll
    for (int k = 0; k < N; k += 4) {
        const float4 a = q_gain ? *reinterpret_cast<const float4*>(q_gain + c * N + k) : make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 b = k_gain ? *reinterpret_cast<const float4*>(k_gain + c * N + k) : make_float4(1.f, 1.f, 1.f, 1.f);
        gq[k] = a.x; gq[k + 1] = a.y; gq[k + 2] = a.z; gq[k + 3] = a.w;
        gk[k] = b.x; gk[k + 1] = b.y; gk[k + 2] = b.z; gk[k + 3] = b.w;
    }
    // where this token's keys and values go
    const int slot = slots[t];
    const bool write_kv = k_pool && slot >= 0;
    int page = 0, off = 0;
    if (write_kv) {
        page = slot / page_size; off = slot % page_size;
        if (page >= n_pages) { if (lane == 0) atomicOr(status, 2); return; }
    }
    const int xr = swizzle ? (off & 7) : 0;
    const T* src = qkv + (size_t)t * heads * HD + c * N;
    pdl_wait(KID_QK);
    for (int h0 = warp * HPW * UNR; h0 < heads; h0 += warps * HPW * UNR) {
        Vec16<T> v[UNR];
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            const int h = h0 + u * HPW + sub;
            v[u].load(src + (size_t)(h < heads ? h : heads - 1) * HD);
        }
#pragma unroll
        for (int u = 0; u < UNR; u++) {
            const int h = h0 + u * HPW + sub;
            if (h0 + u * HPW >= heads) break;          // the whole warp is past the last head
            const bool live = h < heads;
            const bool is_q = h < nh, is_k = !is_q && h < nh + nkv;
            float f[N];
            v[u].unpack(f);
            float ss = 0.f;
#pragma unroll
            for (int k = 0; k < N; k++) ss += f[k] * f[k];
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if ((is_q && q_gain) || (is_k && k_gain)) {
                const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
                for (int k = 0; k < N; k++) f[k] = f[k] * inv * (is_q ? gq[k] : gk[k]);
            }
            if (cos_t) {
#pragma unroll
                for (int k = 0; k < N; k++) {
                    const float other = __shfl_xor_sync(0xffffffffu, f[k], LPH / 2);
                    // upper half: x cos + partner sin; lower half: x cos - partner sin (the sign is in sn)
                    if (is_q || is_k) f[k] = f[k] * cs[k] + other * sn[k];
                }
            }
            if (!live) continue;
            T* dst;
            int x = 0;
            if (is_q) {
                dst = q_out + (size_t)t * nh * HD + (size_t)h * HD;
            } else {
                if (!write_kv) continue;
                const int kh = is_k ? h - nh : h - nh - nkv;
                dst = (is_k ? k_pool : v_pool) + (((size_t)page * nkv + kh) * page_size + off) * HD;
                x = xr;
            }
            Vec16<T> o;
            o.pack(f);
            o.store(dst + (c ^ x) * N);
        }
    }
}

// From how many tokens on a CTA takes a whole token (a setter for tuning runs).  Measured back to back in a
// captured loop, 16 + 2 x 8 heads of 128, microseconds a CTA a token / a warp a pair of heads: 128 tokens
// 3.6 / 3.2, 256: 4.2 / 4.5, 512: 4.4 / 5.0, 1024: 5.7 / 7.5, 2048: 9.8 / 12.1, 4096: 17.8 / 21.8.
static int g_qk_token_threshold = 256;
PLLM_EXPORT int pllm_qk_set_token_threshold(int n) {
    const int was = g_qk_token_threshold;
    g_qk_token_threshold = n;
    return was;
}

template <typename T, int LPH>
static void launch_qk_vec(const void* qkv, void* q_out, const float* q_gain, const float* k_gain, float eps,
                          const float* cos_t, const float* sin_t, int max_pos, const int* positions, const int* slots,
                          void* k_pool, void* v_pool, int n_tokens, int nh, int nkv, int page_size, int n_pages,
                          int swizzle, int* status, cudaStream_t stream) {
    const long long items = (long long)n_tokens * (nh + 2 * nkv);
    const int per_block = 4 * (32 / LPH);
    if (n_tokens >= g_qk_token_threshold) {
        // enough tokens to fill the GPU with a warp each
        launch_chained(qk_norm_rope_kv_token_kernel<T, LPH>, dim3((unsigned)n_tokens), dim3(128), 0, stream,
                       (const T*)qkv, (T*)q_out, q_gain, k_gain, eps, cos_t, sin_t, max_pos, positions, slots, (T*)k_pool,
                       (T*)v_pool, n_tokens, nh, nkv, page_size, n_pages, swizzle, status);
        return;
    }
    launch_chained(qk_norm_rope_kv_vec_kernel<T, LPH>, dim3((unsigned)((items + per_block - 1) / per_block)), dim3(128), 0,
                   stream, (const T*)qkv, (T*)q_out, q_gain, k_gain, eps, cos_t, sin_t, max_pos, positions, slots,
                   (T*)k_pool, (T*)v_pool, n_tokens, nh, nkv, page_size, n_pages, swizzle, status);
}

PLLM_EXPORT int pllm_qk_norm_rope_kv(int dtype, const void* qkv, void* q_out, const float* q_gain,
                                     const float* k_gain, float eps, const float* cos_t, const float* sin_t,
                                     int rotary_dim, int max_pos, const int* positions, const int* slots,
                                     void* k_pool, void* v_pool, int n_tokens, int nh, int nkv, int hd,
                                     int page_size, int n_pages, int swizzle, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return PLLM_OK;
    // a swizzled row needs a whole number of 8-chunk groups
    if (swizzle && (hd * (dtype == PLLM_F32 ? 4 : 2) / 16) % 8 != 0) return PLLM_ERR_SIZE;
    if (nh <= 0 || nkv < 0 || hd <= 0 || page_size <= 0) return PLLM_ERR_SIZE;
    if (cos_t && (rotary_dim <= 0 || rotary_dim > hd || (rotary_dim & 1))) return PLLM_ERR_SIZE;
    // sixteen bytes a lane where the head is 8, 16 or 32 chunks wide and rotated over its whole width
    const int chunks = hd * (dtype == PLLM_F32 ? 4 : 2) / 16;
    if ((dtype == PLLM_F32 || dtype == PLLM_BF16) && (chunks == 8 || chunks == 16 || chunks == 32) &&
        hd * (dtype == PLLM_F32 ? 4 : 2) % 16 == 0 && (!cos_t || rotary_dim == hd)) {
#define PLLM_QK_VEC(T, LPH)                                                                                        \
    launch_qk_vec<T, LPH>(qkv, q_out, q_gain, k_gain, eps, cos_t, sin_t, max_pos, positions, slots, k_pool, v_pool, \
                          n_tokens, nh, nkv, page_size, n_pages, swizzle, status, stream)
        if (dtype == PLLM_F32) {
            if (chunks == 8) PLLM_QK_VEC(float, 8); else if (chunks == 16) PLLM_QK_VEC(float, 16); else PLLM_QK_VEC(float, 32);
        } else {
            if (chunks == 8) PLLM_QK_VEC(bf16, 8); else if (chunks == 16) PLLM_QK_VEC(bf16, 16); else PLLM_QK_VEC(bf16, 32);
        }
#undef PLLM_QK_VEC
        return launch_status();
    }
    const int warps = 4;
    const size_t smem = (size_t)warps * hd * sizeof(float);
    if (smem > 48 * 1024) return PLLM_ERR_LIMIT;
    const long long items = (long long)n_tokens * (nh + 2 * nkv);
    const int blocks = (int)((items + warps - 1) / warps);
    PLLM_DISPATCH_DTYPE(dtype, {
        launch_chained(qk_norm_rope_kv_kernel<T>, dim3(blocks), dim3(warps * 32), smem, stream,
                       (const T*)qkv, (T*)q_out, q_gain, k_gain, eps, cos_t, sin_t, rotary_dim, max_pos, positions, slots,
                       (T*)k_pool, (T*)v_pool, n_tokens, nh, nkv, hd, page_size, n_pages, swizzle, status);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(qk_norm_rope_kv)

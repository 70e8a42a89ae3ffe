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
    const T* __restrict__ qkv,        // [n_tokens, (nh + 2*nkv) * hd]
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
    pdl_wait();
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

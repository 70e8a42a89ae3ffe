// Paged attention for any head size (a multiple of 4 floats / 8 bfloat16 up to
// 256), any number of heads and groups, any page size, with an optional window:
// the kernel of the true 32-bit path, and of bfloat16 shapes that the tuned
// kernels do not take.  Arithmetic in float on the CUDA cores.
//
// What it computes is the reference's attention
// (crates/pagedllm/src/model/attention.rs:198-214 and
// crates/pagedllm/src/kernels/paged_attention.cu:86-147): for query head h the
// keys and values of kv head h / group; score = q.k * scale; key j is visible to
// the query at position p iff j <= p (and, with a window w, j > p - w);
// softmax in float; weighted sum of values.  Unlike the reference's kernel it
// keeps no score buffer as long as the context: the softmax runs online over
// tiles of 32 keys, so the context is bounded by the cache alone.
//
// Work comes as a list of items prepared on the host, one CTA per (item, kv
// head, part of the group):
//   item = {seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split}
// q_count consecutive tokens of one request (token index q_token0.. in the step,
// positions q_pos0..) attend over keys [kv_begin, kv_end) of the request's block
// table row `seg`.  part_slot < 0: the item sees all keys its queries may see and
// writes the normalised output.  part_slot >= 0: the item is one split of a long
// key range and writes (max, sum, unnormalised output) for attention_reduce.
#include "common.cuh"

#define ATT_BK 32        // keys per tile
#define ATT_MAX_ROWS 16  // query rows (token x head of the group) per CTA, one warp each
#define ATT_MAX_HD 256

struct AttnWork { int seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split; };   // split: count << 16 | index (0: not split)

template <typename T>
__global__ void attention_generic_kernel(
    // q and the pools are written by the kernels before this one: not __restrict__, so that they are
    // read with coherent loads after the wait and never through the read-only cache
    const T* q,            // [n_tokens, nh, hd]
    const T* k_pool, const T* v_pool,  // [pages, nkv, page_size, hd]
    const int* __restrict__ block_tables,  // [n_segs, table_width]
    const AttnWork* __restrict__ work, const int* __restrict__ n_work_ptr,
    T* __restrict__ out,                // [n_tokens, nh, hd]
    float* __restrict__ part_o,         // [parts, nh, hd]
    float* __restrict__ part_ml,        // [parts, nh, 2]
    int nh, int nkv, int hd, int page_size, int n_pages, int table_width, int window, float scale,
    int heads_per_cta, int* status) {
    pdl_launch_dependents();
    pdl_wait(KID_ATT_GENERIC);
    if ((int)blockIdx.x >= *n_work_ptr) return;
    const AttnWork w = work[blockIdx.x];
    const int group = nh / nkv;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    const int kh = blockIdx.y / gparts;
    const int head0 = kh * group + (blockIdx.y % gparts) * heads_per_cta;       // first q head of this CTA
    const int n_heads = min(heads_per_cta, kh * group + group - head0);
    const int rows = w.q_count * n_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int hdp = hd + 4;  // padded row: conflict-free float4 reads across keys

    extern __shared__ float smem[];
    float* q_s = smem;                               // [ATT_MAX_ROWS][hd]
    float* k_s = q_s + ATT_MAX_ROWS * hd;            // [ATT_BK][hdp]
    float* v_s = k_s + ATT_BK * hdp;                 // [ATT_BK][hdp]
    __shared__ int page_s[ATT_BK];

    // Row r of the CTA: token r / n_heads of the item, head head0 + r % n_heads.
    const bool active = warp < rows;
    const int tq = active ? warp / n_heads : 0;
    const int head = active ? head0 + warp % n_heads : head0;
    const int pos = w.q_pos0 + tq;
    if (active) {
        const T* qr = q + ((size_t)(w.q_token0 + tq) * nh + head) * hd;
        for (int e = lane; e < hd; e += 32) q_s[warp * hd + e] = to_f32(qr[e]) * scale;
    }
    // Keys this row may see inside the item's range.
    const int lo = max(w.kv_begin, window > 0 ? pos - window + 1 : 0);
    const int hi = min(w.kv_end, pos + 1);

    float m = -CUDART_INF_F, l = 0.f;
    float acc[ATT_MAX_HD / 32];
#pragma unroll
    for (int k = 0; k < ATT_MAX_HD / 32; k++) acc[k] = 0.f;

    constexpr int N = Vec16<T>::N;
    const int vec_per_row = hd / N;
    const int* table = block_tables + (size_t)w.seg * table_width;

    for (int kv0 = w.kv_begin; kv0 < w.kv_end; kv0 += ATT_BK) {
        __syncthreads();  // the previous tile is no longer read
        if (threadIdx.x < ATT_BK) {
            const int j = kv0 + threadIdx.x;
            int page = -1;
            if (j < w.kv_end) {
                const int b = j / page_size;
                page = b < table_width ? table[b] : -1;
                // A freed page of a window layer holds -1 and is never visible to a
                // query of this item; anything else out of range is a fault.
                if (page >= n_pages) { atomicOr(status, 8); page = -1; }
            }
            page_s[threadIdx.x] = page;
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < ATT_BK * vec_per_row; idx += blockDim.x) {
            const int j = idx / vec_per_row, c = (idx % vec_per_row) * N;
            const int page = page_s[j];
            float fk[N], fv[N];
            if (page >= 0) {
                const size_t base = (((size_t)page * nkv + kh) * page_size + (kv0 + j) % page_size) * hd + c;
                Vec16<T> vk, vv;
                vk.load(k_pool + base); vv.load(v_pool + base);
                vk.unpack(fk); vv.unpack(fv);
            } else {
#pragma unroll
                for (int k = 0; k < N; k++) { fk[k] = 0.f; fv[k] = 0.f; }
            }
#pragma unroll
            for (int k = 0; k < N; k++) { k_s[j * hdp + c + k] = fk[k]; v_s[j * hdp + c + k] = fv[k]; }
        }
        __syncthreads();
        if (!active) continue;
        const int j = kv0 + lane;
        const bool visible = j >= lo && j < hi;
        if (!__any_sync(0xffffffffu, visible)) continue;
        float s = 0.f;
        {
            const float4* kr = reinterpret_cast<const float4*>(k_s + lane * hdp);
            const float4* qr = reinterpret_cast<const float4*>(q_s + warp * hd);
            for (int c = 0; c < hd / 4; c++) {
                const float4 a = qr[c], b = kr[c];
                s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
            }
        }
        s = visible ? s : -CUDART_INF_F;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = visible ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);  // m = -inf on the first visible tile: exp(-inf) = 0
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int k = 0; k < ATT_MAX_HD / 32; k++) acc[k] *= corr;
        for (int jj = 0; jj < ATT_BK; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            if (pj == 0.f) continue;  // uniform across the warp
            const float* vr = v_s + jj * hdp;
#pragma unroll
            for (int k = 0; k < ATT_MAX_HD / 32; k++)
                if (k * 32 + lane < hd) acc[k] = fmaf(pj, vr[k * 32 + lane], acc[k]);
        }
    }
    if (!active) return;
    if (w.part_slot < 0) {
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        T* o = out + ((size_t)(w.q_token0 + tq) * nh + head) * hd;
#pragma unroll
        for (int k = 0; k < ATT_MAX_HD / 32; k++)
            if (k * 32 + lane < hd) o[k * 32 + lane] = from_f32<T>(acc[k] * inv);
    } else {
        const size_t pr = (size_t)(w.part_slot + tq) * nh + head;
        float* o = part_o + pr * hd;
#pragma unroll
        for (int k = 0; k < ATT_MAX_HD / 32; k++)
            if (k * 32 + lane < hd) o[k * 32 + lane] = acc[k];
        if (lane == 0) { part_ml[pr * 2] = m; part_ml[pr * 2 + 1] = l; }
    }
}

// Combine the splits of a token: for entry t,
// red[t] = {token, first, count, stride}: its parts are first + s * stride, s < count.
// One CTA per (entry, head), RED_GROUPS groups of hd threads.  The weights exp(m_s - M) are
// formed once in shared memory (one warp, every split's (m, l) fetched in one trip); then group
// g sums the splits s = g, g + RED_GROUPS, ... of its output dimension, all its loads in flight
// together, and the groups' sums are added in the order of the groups: always the same order,
// whatever ran where.
#define RED_MAX_SPLITS 256
#define RED_GROUPS 4
template <typename T>
__global__ void attention_reduce_kernel(const float* part_o, const float* part_ml,   // just written: no __restrict__
                                        const int* __restrict__ red, const int* __restrict__ n_red_ptr,
                                        T* __restrict__ out, int nh, int hd) {
    __shared__ float wgt[RED_MAX_SPLITS];
    __shared__ float inv_s;
    extern __shared__ float gsum[];     // [RED_GROUPS][hd]
    pdl_launch_dependents();
    // The list of reductions is the host's (part of the step's packed buffer): how many there are and this
    // CTA's first entry are fetched before the wait for the attention kernel, two trips to L2 that then
    // lie beside that kernel's end and not behind it.
    const int head = blockIdx.y, n_red = *n_red_ptr;
    int4 entry = make_int4(0, 0, 0, 0);
    if ((int)blockIdx.x < n_red) entry = make_int4(red[blockIdx.x * 4], red[blockIdx.x * 4 + 1], red[blockIdx.x * 4 + 2], red[blockIdx.x * 4 + 3]);   // (the list need not lie on a 16-byte boundary)
    pdl_wait(KID_ATT_REDUCE);
    const int ng = blockDim.x / hd;                               // groups of hd threads: 1 or RED_GROUPS
    const int grp = threadIdx.x / hd, d = threadIdx.x % hd;
    // a CTA takes entries blockIdx.x, blockIdx.x + gridDim.x, ...: a captured step launches a grid for
    // the most entries a step could have, and CTAs with nothing to do must be few
    for (int t = blockIdx.x; t < n_red; t += gridDim.x) {
        if (t != (int)blockIdx.x) entry = make_int4(red[t * 4], red[t * 4 + 1], red[t * 4 + 2], red[t * 4 + 3]);
        const int token = entry.x, first = entry.y, count = min(entry.z, RED_MAX_SPLITS), stride = entry.w;
        if (count <= 0) continue;
        if (count <= 8 && ng == 1) {
            // few splits (the usual case away from batch 1): every thread fetches the entry's (m, l) pairs and
            // its own column of the partial rows in one trip, nothing goes through shared memory and no
            // thread waits for another, so a CTA's entries follow one another at the pace of the loads
            float2 ml[8];
            float v[8], M = -CUDART_INF_F;
            const float* po = part_o + ((size_t)first * nh + head) * hd + d;
            const size_t s_stride = (size_t)stride * nh * hd;
#pragma unroll
            for (int s = 0; s < 8; s++) {
                ml[s] = make_float2(-CUDART_INF_F, 0.f);
                v[s] = 0.f;
                if (s < count) {
                    ml[s] = *reinterpret_cast<const float2*>(part_ml + ((size_t)(first + s * stride) * nh + head) * 2);
                    v[s] = po[(size_t)s * s_stride];
                }
                M = fmaxf(M, ml[s].x);
            }
            float L = 0.f, o = 0.f;
#pragma unroll
            for (int s = 0; s < 8; s++) {
                if (s >= count) break;
                const float f = ml[s].x == -CUDART_INF_F ? 0.f : expf(ml[s].x - M);
                L += ml[s].y * f;
                o = fmaf(v[s], f, o);
            }
            out[((size_t)token * nh + head) * hd + d] = from_f32<T>(o * (L > 0.f ? 1.0f / L : 0.f));
            continue;
        }
        __syncthreads();       // the weights and sums of the entry before are no longer read
        if (threadIdx.x < 32) {
            // up to 8 splits a lane, their (m, l) pairs fetched together
            float2 ml[RED_MAX_SPLITS / 32];
            float M = -CUDART_INF_F;
#pragma unroll
            for (int i = 0; i < RED_MAX_SPLITS / 32; i++) {
                const int s = threadIdx.x + 32 * i;
                ml[i] = make_float2(-CUDART_INF_F, 0.f);
                if (s < count) ml[i] = *reinterpret_cast<const float2*>(part_ml + ((size_t)(first + s * stride) * nh + head) * 2);
                M = fmaxf(M, ml[i].x);
            }
            M = warp_max(M);
            float L = 0.f;
#pragma unroll
            for (int i = 0; i < RED_MAX_SPLITS / 32; i++) {
                const int s = threadIdx.x + 32 * i;
                if (s >= count) continue;
                const float f = ml[i].x == -CUDART_INF_F ? 0.f : expf(ml[i].x - M);
                wgt[s] = f;
                L += ml[i].y * f;
            }
            L = warp_sum(L);
            if (threadIdx.x == 0) inv_s = L > 0.f ? 1.0f / L : 0.f;
        }
        __syncthreads();
        {
            const float* po = part_o + ((size_t)first * nh + head) * hd + d;
            const size_t s_stride = (size_t)stride * nh * hd;
            float o = 0.f;
            for (int s0 = grp; s0 < count; s0 += ng * 4) {
                float v[4];
#pragma unroll
                for (int i = 0; i < 4; i++) v[i] = s0 + i * ng < count ? po[(size_t)(s0 + i * ng) * s_stride] : 0.f;
#pragma unroll
                for (int i = 0; i < 4; i++)
                    if (s0 + i * ng < count) o = fmaf(v[i], wgt[s0 + i * ng], o);
            }
            gsum[grp * hd + d] = o;
        }
        __syncthreads();
        if (grp == 0) {
            float o = gsum[d];
#pragma unroll
            for (int g2 = 1; g2 < RED_GROUPS; g2++)
                if (g2 < ng) o += gsum[g2 * hd + d];
            out[((size_t)token * nh + head) * hd + d] = from_f32<T>(o * inv_s);
        }
    }
}

PLLM_EXPORT int pllm_attention_generic(int dtype, const void* q, const void* k_pool, const void* v_pool,
                                       const int* block_tables, const int* work, const int* n_work_ptr,
                                       int max_work, void* out, float* part_o, float* part_ml, int nh, int nkv,
                                       int hd, int page_size, int n_pages, int table_width, int window,
                                       float scale, int* status, cudaStream_t stream) {
    if (max_work <= 0) return PLLM_OK;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || page_size <= 0) return PLLM_ERR_SIZE;
    if (hd <= 0 || hd > ATT_MAX_HD || hd % 8 != 0) return PLLM_ERR_SIZE;
    const int group = nh / nkv;
    const int heads_per_cta = group < ATT_MAX_ROWS ? group : ATT_MAX_ROWS;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    const size_t smem = ((size_t)ATT_MAX_ROWS * hd + 2 * (size_t)ATT_BK * (hd + 4)) * sizeof(float);
    PLLM_DISPATCH_DTYPE(dtype, {
        cudaFuncSetAttribute(attention_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        dim3 grid(max_work, nkv * gparts);
        launch_chained(attention_generic_kernel<T>, grid, dim3(ATT_MAX_ROWS * 32), smem, stream,
                       (const T*)q, (const T*)k_pool, (const T*)v_pool, block_tables, (const AttnWork*)work, n_work_ptr,
                       (T*)out, part_o, part_ml, nh, nkv, hd, page_size, n_pages, table_width, window, scale,
                       heads_per_cta, status);
    });
    return launch_status();
}

// The most query tokens one work item may hold for a given group size, so that
// the host cuts tiles the kernel accepts.
PLLM_EXPORT int pllm_attention_generic_tile_tokens(int nh, int nkv) {
    const int group = nh / nkv;
    const int heads_per_cta = group < ATT_MAX_ROWS ? group : ATT_MAX_ROWS;
    return ATT_MAX_ROWS / heads_per_cta;
}

// many_splits: the entries have eight splits or more each (a step of very few tokens): four groups of
// threads share an entry's splits; else one group (measured, 0.6B shape: batch 1, 16 splits: 0.911
// against 0.933 ms a step with four; batch 8, 4 splits: 1.503 against 1.478).
PLLM_EXPORT int pllm_attention_reduce(int dtype, const float* part_o, const float* part_ml, const int* red,
                                      const int* n_red_ptr, int max_red, void* out, int nh, int hd, int many_splits,
                                      cudaStream_t stream) {
    if (max_red <= 0) return PLLM_OK;
    const int groups = many_splits && RED_GROUPS * hd <= 1024 ? RED_GROUPS : 1;
    PLLM_DISPATCH_DTYPE(dtype, {
        // (a captured step launches its capacity, and every CTA of it costs its start even with nothing to do:
        // 256 x heads instead of 64 cost the 2048-token step 4 us a layer; the CTAs loop over the entries)
        dim3 grid(max_red < 64 ? max_red : 64, nh);
        launch_chained(attention_reduce_kernel<T>, grid, dim3(groups * hd), (size_t)groups * hd * sizeof(float), stream,
                       part_o, part_ml, red,
                       n_red_ptr, (T*)out, nh, hd);
    });
    return launch_status();
}

PLLM_TRACE_EXPORT(attention_generic)

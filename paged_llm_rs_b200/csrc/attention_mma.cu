// Paged attention in bfloat16 on the tensor cores, head sizes 64 and 128: the
// serving kernel for prefill portions and for decoding.
//
// Same arithmetic as attention_generic.cu (the reference's
// crates/pagedllm/src/model/attention.rs:198-214 and
// crates/pagedllm/src/kernels/paged_attention.cu:86-147): scores q.k * scale over
// the keys a query may see, softmax in float, weighted sum of values; query head
// h reads kv head h / group.  Unlike the reference's kernel, which re-reads every
// key once per query head and keeps a score buffer as long as the context, one
// CTA serves all query heads of a kv head from one copy of the keys and values
// in shared memory, and the softmax runs online.
//
// One CTA (4 warps) per (work item, kv head, part of the group).  Work items are
// the ones attention_plan.py cuts (see attention_generic.cu for the layout).
// Keys and values are brought page by page into a 3-stage ring of 64-key tiles
// with cp.async (16 bytes a thread, rows past the range or in pages that were
// given back are zero-filled), read with ldmatrix from a swizzled layout, and
// multiplied with mma.sync.m16n8k16 (bf16 in, float accumulate).
//
//   items of several query tokens: rows (token, head) of the tile are spread over the
//       warps, 16 rows each; all warps walk the same key tiles.
//   items of one query token (decoding): the heads of the group are the rows of ONE
//       16-row block; the four warps take 16 keys each of every 64-key tile with a
//       running (max, sum, output) of their own, combined through shared memory at
//       the end.
#include "common.cuh"

#define MMA_BK 64
#define MMA_STAGES 3
#define MMA_ROWS 64

struct AttnWork { int seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split; };   // split: count << 16 | index (0: not split)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows are HD
// bfloat16 wide; chunks are XOR-swizzled with the row so that the 8 rows an
// ldmatrix reads at one chunk index fall into different banks.
template <int HD> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

template <int HD>
struct TileLoader {
    // Loads keys [kv0, kv0 + MMA_BK) of the item into one stage.  Thread t copies chunk
    // t % CH of rows t / CH + k * RPP.
    static constexpr int CH = HD / 8;             // 16-byte chunks a row
    static constexpr int RPP = 128 / CH;          // rows a pass of the CTA covers
    static constexpr int PASSES = MMA_BK / RPP;
    const bf16* k_pool; const bf16* v_pool; const int* table;
    int table_width, page_size, page_shift, n_pages, nkv, kh, kv_end, swizzle_mask;  // mask 7: swizzled cache, 0: plain

    __device__ __forceinline__ void load(uint32_t k_s, uint32_t v_s, int kv0, int* status) const {
        const int chunk = threadIdx.x % CH, r0 = threadIdx.x / CH;
#pragma unroll
        for (int p = 0; p < PASSES; p++) {
            const int row = r0 + p * RPP;
            const int j = kv0 + row;
            bool valid = j < kv_end;
            size_t base = 0;
            if (valid) {
                const int b = page_shift >= 0 ? (j >> page_shift) : (j / page_size);
                const int o = j - b * page_size;
                int page = b < table_width ? table[b] : -1;
                if (page >= n_pages) { atomicOr(status, 8); page = -1; }
                valid = page >= 0;
                // a swizzled cache keeps logical chunk c of a row at c ^ (offset in page & 7)
                base = (((size_t)(valid ? page : 0) * nkv + kh) * page_size + o) * HD + ((chunk ^ (o & swizzle_mask)) * 8);
            }
            const uint32_t off = tile_off<HD>(row, chunk);
            cp_async16(k_s + off, k_pool + base, valid);
            cp_async16(v_s + off, v_pool + base, valid);
        }
    }
};

template <int HD>
__global__ void __launch_bounds__(128, 2) attention_mma_kernel(
    const bf16* q, const bf16* k_pool, const bf16* v_pool,   // written by the kernels before this one: no __restrict__
    const int* __restrict__ block_tables, const AttnWork* __restrict__ work, const int* __restrict__ n_work_ptr,
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    int nh, int nkv, int page_size, int page_shift, int n_pages, int table_width, int window, float scale_log2,
    int heads_per_cta, int swizzle, int kinds_mask, int* status) {
    pdl_wait(KID_ATT_MMA);
    if ((int)blockIdx.y >= *n_work_ptr) return;
    const AttnWork w = work[blockIdx.y];
    const int group = nh / nkv;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    const int kh = blockIdx.x / gparts;
    const int head0 = kh * group + (blockIdx.x % gparts) * heads_per_cta;
    const int n_heads = min(heads_per_cta, kh * group + group - head0);
    const int rows = w.q_count * n_heads;          // <= MMA_ROWS
    const bool decode = w.q_count == 1;            // one token: the warps split the keys, not the rows
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int CH = HD / 8;
    constexpr int KSTEPS = HD / 16;                // k-steps of q.k^T
    constexpr int DTILES = HD / 8;                 // 8-wide output tiles of p.v
    constexpr int STAGE_BYTES = 2 * MMA_BK * HD * 2;

    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t smem_base = smem_u32(smem);

    TileLoader<HD> loader{k_pool, v_pool, block_tables + (size_t)w.seg * table_width, table_width, page_size, page_shift,
                          n_pages, nkv, kh, w.kv_end, swizzle ? 7 : 0};
    if (!(kinds_mask & (w.q_count == 1 ? 1 : 2))) return;   // the bulk-copy kernel takes these items

    // ---- q rows into a buffer of their own; the first key tiles are requested at once --------
    const uint32_t q_s = smem_base + MMA_STAGES * STAGE_BYTES;
    for (int idx = threadIdx.x; idx < (decode ? 16 : MMA_ROWS) * CH; idx += 128) {
        const int row = idx / CH, chunk = idx % CH;
        const bool valid = row < rows;
        const int tq = valid ? row / n_heads : 0, hg = valid ? row % n_heads : 0;
        const bf16* src = q + ((size_t)(w.q_token0 + tq) * nh + head0 + hg) * HD + chunk * 8;
        cp_async16(q_s + tile_off<HD>(row, chunk), src, valid);
    }
    cp_async_commit();
    const int n_tiles = (w.kv_end - w.kv_begin + MMA_BK - 1) / MMA_BK;
#pragma unroll
    for (int s = 0; s < MMA_STAGES - 1; s++) {
        if (s < n_tiles) loader.load(smem_base + s * STAGE_BYTES, smem_base + s * STAGE_BYTES + MMA_BK * HD * 2,
                                     w.kv_begin + s * MMA_BK, status);
        cp_async_commit();
    }
    cp_async_wait<MMA_STAGES - 1>();   // q has landed; the key tiles may still be in flight
    __syncthreads();
    uint32_t qf[KSTEPS][4];
    {
        const int rbase = decode ? 0 : warp * 16;
        const int mat = lane >> 3;
        const int row = rbase + (lane & 7) + (mat & 1) * 8;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) ldmatrix_x4(qf[ks], q_s + tile_off<HD>(row, ks * 2 + (mat >> 1)));
    }

    // ---- the two rows of this thread and what they may see -----------------------------------
    const int r0 = (decode ? 0 : warp * 16) + (lane >> 2), r1 = r0 + 8;
    int lo[2], hi[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = i ? r1 : r0;
        if (r < rows) {
            const int pos = w.q_pos0 + r / n_heads;
            lo[i] = max(w.kv_begin, window > 0 ? pos - window + 1 : 0);
            hi[i] = min(w.kv_end, pos + 1);
        } else { lo[i] = 0; hi[i] = 0; }
    }
    // keys beyond every row of the warp need no arithmetic
    int warp_hi = max(hi[0], hi[1]), warp_lo = min(hi[0] > lo[0] ? lo[0] : 0x7fffffff, hi[1] > lo[1] ? lo[1] : 0x7fffffff);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        warp_hi = max(warp_hi, __shfl_xor_sync(0xffffffffu, warp_hi, o));
        warp_lo = min(warp_lo, __shfl_xor_sync(0xffffffffu, warp_lo, o));
    }

    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
    float o_acc[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; d++) { o_acc[d][0] = o_acc[d][1] = o_acc[d][2] = o_acc[d][3] = 0.f; }

    // keys of a tile this warp multiplies: all 64 (several query tokens) or its own 16 (decoding)
    const int key_base = decode ? warp * 16 : 0;
    const int NT = decode ? 2 : 8;   // 8-key score tiles per warp and key tile

    for (int t = 0; t < n_tiles; t++) {
        cp_async_wait<MMA_STAGES - 2>();
        __syncthreads();
        {
            const int nt = t + MMA_STAGES - 1;
            if (nt < n_tiles) {
                const uint32_t sb = smem_base + (nt % MMA_STAGES) * STAGE_BYTES;
                loader.load(sb, sb + MMA_BK * HD * 2, w.kv_begin + nt * MMA_BK, status);
            }
            cp_async_commit();
        }
        const int kv0 = w.kv_begin + t * MMA_BK;
        if (kv0 + key_base >= warp_hi || kv0 + key_base + NT * 8 <= warp_lo) continue;
        const uint32_t k_s = smem_base + (t % MMA_STAGES) * STAGE_BYTES, v_s = k_s + MMA_BK * HD * 2;

        // ---- scores: S[16 rows][NT*8 keys] ---------------------------------------------
        float s_acc[8][4];
#pragma unroll
        for (int n = 0; n < 8; n++) { s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f; }
        {
            // The asm statements run in the order written.  One k-step at a time over all
            // key tiles: the fragments of a step are fetched together, and neighbouring
            // mma write different accumulators, so none waits for the one before it.
            const int mat = lane >> 3;
            const int np_count = NT / 2;
            const int key0 = key_base + (lane & 7) + (mat >> 1) * 8;
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) {
                uint32_t kf[4][4];
#pragma unroll
                for (int np = 0; np < 4; np++)
                    if (np < np_count) ldmatrix_x4(kf[np], k_s + tile_off<HD>(key0 + np * 16, ks * 2 + (mat & 1)));
#pragma unroll
                for (int np = 0; np < 4; np++) {
                    if (np >= np_count) break;
                    mma_bf16(s_acc[np * 2], qf[ks], kf[np][0], kf[np][1]);
                    mma_bf16(s_acc[np * 2 + 1], qf[ks], kf[np][2], kf[np][3]);
                }
            }
        }
        // ---- mask, running max and sum ---------------------------------------------------
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int n = 0; n < 8; n++) {
            if (n >= NT) break;
            const int j = kv0 + key_base + n * 8 + (lane & 3) * 2;
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int jj = j + (e & 1), i = e >> 1;
                const float v = (jj >= lo[i] && jj < hi[i]) ? s_acc[n][e] * scale_log2 : -CUDART_INF_F;
                s_acc[n][e] = v;
                mx[i] = fmaxf(mx[i], v);
            }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int i = 0; i < 2; i++) {
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
            mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
            const float m_new = fmaxf(m_run[i], mx[i]);
            m_use[i] = m_new == -CUDART_INF_F ? 0.f : m_new;   // nothing seen yet: keep exp2 away from inf - inf
            corr[i] = exp2f(m_run[i] - m_use[i]);
            m_run[i] = m_new;
            l_run[i] *= corr[i];
        }
        uint32_t pf[4][4];   // P as A fragments, one per 16 keys
#pragma unroll
        for (int n = 0; n < 8; n++) {
            if (n >= NT) break;
            const float p0 = exp2f(s_acc[n][0] - m_use[0]), p1 = exp2f(s_acc[n][1] - m_use[0]);
            const float p2 = exp2f(s_acc[n][2] - m_use[1]), p3 = exp2f(s_acc[n][3] - m_use[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            pf[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pf[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
#pragma unroll
        for (int d = 0; d < DTILES; d++) {
            o_acc[d][0] *= corr[0]; o_acc[d][1] *= corr[0];
            o_acc[d][2] *= corr[1]; o_acc[d][3] *= corr[1];
        }
        // ---- output += P V ---------------------------------------------------------------------
        {
            const int mat = lane >> 3;
#pragma unroll
            for (int kk = 0; kk < 4; kk++) {          // 16 keys a step
                if (kk * 2 >= NT) break;
                const int key = key_base + kk * 16 + (lane & 7) + (mat & 1) * 8;
                // four fragment loads in flight, then their eight mma
#pragma unroll
                for (int d4 = 0; d4 < DTILES / 2; d4 += 4) {
                    uint32_t vf[4][4];
#pragma unroll
                    for (int i = 0; i < 4; i++)
                        ldmatrix_x4_trans(vf[i], v_s + tile_off<HD>(key, (d4 + i) * 2 + (mat >> 1)));
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        mma_bf16(o_acc[(d4 + i) * 2], pf[kk], vf[i][0], vf[i][1]);
                        mma_bf16(o_acc[(d4 + i) * 2 + 1], pf[kk], vf[i][2], vf[i][3]);
                    }
                }
            }
        }
    }
    cp_async_wait<0>();
    pdl_launch_dependents();   // the key tiles are done: the next kernel's CTAs may take their places
    // row sums live spread over the four lanes of a quad
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }

    if (decode) {
        // ---- combine the four warps' partial results of the same rows ------------------------
        __syncthreads();  // every warp is done reading the ring
        float* o_s = reinterpret_cast<float*>(smem);                 // [4 warps][16 rows][HD]
        float* ml_s = o_s + 4 * 16 * HD;                              // [4][16][2]
#pragma unroll
        for (int d = 0; d < DTILES; d++) {
            const int c = d * 8 + (lane & 3) * 2;
            float* a = o_s + ((size_t)(warp * 16 + (lane >> 2)) * HD + c);
            a[0] = o_acc[d][0]; a[1] = o_acc[d][1];
            a[8 * HD] = o_acc[d][2]; a[8 * HD + 1] = o_acc[d][3];
        }
        if ((lane & 3) == 0) {
            ml_s[(warp * 16 + (lane >> 2)) * 2] = m_run[0]; ml_s[(warp * 16 + (lane >> 2)) * 2 + 1] = l_run[0];
            ml_s[(warp * 16 + (lane >> 2) + 8) * 2] = m_run[1]; ml_s[(warp * 16 + (lane >> 2) + 8) * 2 + 1] = l_run[1];
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < rows * HD; idx += 128) {
            const int r = idx / HD, c = idx % HD;
            float M = -CUDART_INF_F;
#pragma unroll
            for (int wi = 0; wi < 4; wi++) M = fmaxf(M, ml_s[(wi * 16 + r) * 2]);
            float L = 0.f, o = 0.f;
#pragma unroll
            for (int wi = 0; wi < 4; wi++) {
                const float mw = ml_s[(wi * 16 + r) * 2];
                const float f = mw == -CUDART_INF_F ? 0.f : exp2f(mw - M);
                L += ml_s[(wi * 16 + r) * 2 + 1] * f;
                o += o_s[(size_t)(wi * 16 + r) * HD + c] * f;
            }
            const int head = head0 + r;
            if (w.part_slot < 0) {
                out[((size_t)w.q_token0 * nh + head) * HD + c] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
            } else {
                const size_t pr = (size_t)w.part_slot * nh + head;
                part_o[pr * HD + c] = o;
                // partial results carry their maximum in natural-log units, as the generic kernel's do
                if (c == 0) { part_ml[pr * 2] = M * 0.6931471805599453f; part_ml[pr * 2 + 1] = L; }
            }
        }
        return;
    }

#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = i ? r1 : r0;
        if (r >= rows) continue;
        const int tq = r / n_heads, head = head0 + r % n_heads;
        if (w.part_slot < 0) {
            const float inv = l_run[i] > 0.f ? 1.0f / l_run[i] : 0.f;
            bf16* o = out + ((size_t)(w.q_token0 + tq) * nh + head) * HD + (lane & 3) * 2;
#pragma unroll
            for (int d = 0; d < DTILES; d++)
                *reinterpret_cast<uint32_t*>(o + d * 8) = pack_bf16(o_acc[d][i * 2] * inv, o_acc[d][i * 2 + 1] * inv);
        } else {
            const size_t pr = (size_t)(w.part_slot + tq) * nh + head;
            float* o = part_o + pr * HD + (lane & 3) * 2;
#pragma unroll
            for (int d = 0; d < DTILES; d++) { o[d * 8] = o_acc[d][i * 2]; o[d * 8 + 1] = o_acc[d][i * 2 + 1]; }
            if ((lane & 3) == 0) { part_ml[pr * 2] = m_run[i] * 0.6931471805599453f; part_ml[pr * 2 + 1] = l_run[i]; }
        }
    }
}

// Whether the tensor-core kernel takes this shape; the generic kernel takes the rest.
PLLM_EXPORT int pllm_attention_mma_supports(int dtype, int nh, int nkv, int hd) {
    return dtype == PLLM_BF16 && (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0;
}

PLLM_EXPORT int pllm_attention_mma_tile_tokens(int nh, int nkv) {
    const int group = nh / nkv;
    const int heads_per_cta = group < 16 ? group : 16;
    return MMA_ROWS / heads_per_cta;
}

PLLM_EXPORT int pllm_attention_mma(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                   const int* work, const int* n_work_ptr, int max_work, void* out, float* part_o,
                                   float* part_ml, int nh, int nkv, int hd, int page_size, int n_pages,
                                   int table_width, int window, float scale, int swizzle, int kinds_mask,
                                   int* status, cudaStream_t stream) {
    if (max_work <= 0) return PLLM_OK;
    if (!pllm_attention_mma_supports(PLLM_BF16, nh, nkv, hd) || page_size <= 0) return PLLM_ERR_SIZE;
    const int group = nh / nkv;
    const int heads_per_cta = group < 16 ? group : 16;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    int page_shift = -1;
    if ((page_size & (page_size - 1)) == 0) { page_shift = 0; while ((1 << page_shift) < page_size) page_shift++; }
    const float scale_log2 = scale * 1.4426950408889634f;
    dim3 grid(nkv * gparts, max_work);   // heads fastest: the items are dealt to the SMs in the order of the work list
    if (hd == 128) {
        const int smem = MMA_STAGES * 2 * MMA_BK * 128 * 2 + MMA_ROWS * 128 * 2;
        cudaFuncSetAttribute(attention_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        launch_chained(attention_mma_kernel<128>, grid, dim3(128), (size_t)smem, stream,
                       (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_tables, (const AttnWork*)work,
                       n_work_ptr, (bf16*)out, part_o, part_ml, nh, nkv, page_size, page_shift, n_pages, table_width,
                       window, scale_log2, heads_per_cta, swizzle, kinds_mask, status);
    } else {
        const int smem = MMA_STAGES * 2 * MMA_BK * 64 * 2 + MMA_ROWS * 64 * 2;
        cudaFuncSetAttribute(attention_mma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        launch_chained(attention_mma_kernel<64>, grid, dim3(128), (size_t)smem, stream,
                       (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_tables, (const AttnWork*)work,
                       n_work_ptr, (bf16*)out, part_o, part_ml, nh, nkv, page_size, page_shift, n_pages, table_width,
                       window, scale_log2, heads_per_cta, swizzle, kinds_mask, status);
    }
    return launch_status();
}

PLLM_TRACE_EXPORT(attention_mma)

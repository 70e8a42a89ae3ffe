// Attention of a prompt portion over the paged cache on the fifth-generation tensor cores.
//
// What it computes is the reference's attention (scores, causal mask over absolute
// positions, float softmax, weighted sum: crates/pagedllm/src/model/attention.rs:190-214 and
// crates/pagedllm/src/kernels/paged_attention.rs:114-188), for work items of several query
// tokens (kernels/attention_plan.py).  A CTA takes one item and one kv head: up to 128 rows
// = query tokens x the heads of the group, and walks the item's keys 64 at a time:
//
//   S = Q K^T     tcgen05.mma, 128 x 64, Q and the key tile in shared memory, S in tensor memory
//   P = softmax   four warps, ONE ROW A THREAD (a thread's lane of tensor memory is its row, so
//                 the row's maximum and sum need no shuffles): tcgen05.ld, scale, mask, exp2,
//                 P rounded to bfloat16 into shared memory in the tensor cores' layout
//   O += P V      tcgen05.mma, 128 x head_dim, O stays in tensor memory for the whole item
//
// Six warps: 0-3 softmax and epilogue, 4 the producer (TMA), 5 allocates tensor memory and
// one of its lanes issues every tcgen05.mma.  S has two buffers, so the tensor cores form
// the next tile's scores while the warps work on this one's; the rows' running maximum is
// only moved when it grew by more than 2^8 (then O is rescaled in tensor memory), which is
// exact after the final division and keeps the tensor memory traffic off the common path.
//
// Shared-memory layouts.  A tile for the tensor cores has rows of 128 bytes (64 values) with
// the 128-byte swizzle (tcgen05.cuh).  The cache stores a key's or value's row (head_dim
// values) with its 16-byte chunk c at c ^ (offset in page & 7), which within each half of 64
// values IS that swizzle; so a page's rows are fetched by TMA tile loads WITHOUT hardware
// swizzle, one per half, and land as planes [64 keys][64 values] the tensor cores read
// directly: K-major for Q K^T, MN-major (rows are the k of the product) for P V.  Q comes
// from the step's plain [tokens, heads, head_dim] buffer through a three-dimensional map
// with the hardware swizzle.
//
// Every wait is bounded (status bit 128 when one ran out).
#include "tcgen05.cuh"

using namespace tc;

struct AttnWork { int seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split; };

namespace {

constexpr int P_ROWS = 128, P_BK = 64, P_STAGES = 5, P_THREADS = 192;
constexpr int P_PLANE = P_BK * 128;            // 64 keys x 128 bytes
constexpr float P_RESCALE = 8.0f;              // log2 units the running maximum may lag behind

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace

template <int HD>
__global__ void __launch_bounds__(P_THREADS, 1) attention_prefill_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_tables, const AttnWork* __restrict__ work,
    const int* __restrict__ n_work_ptr, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    int nh, int nkv, int page_size, int page_shift, int n_pages, int table_width, float scale_log2, int heads_per_cta,
    int tile_tokens, int* status) {
    constexpr int NHALF = HD / 64;
    constexpr int Q_BYTES = NHALF * P_ROWS * 128, STAGE = 2 * NHALF * P_PLANE, P_BYTES = P_ROWS * 128;
    constexpr uint32_t TMEM_COLS = 256, S_COL = 0, O_COL = 128;
    if ((int)blockIdx.y >= *n_work_ptr) return;
    const AttnWork w = work[blockIdx.y];
    if (w.q_count <= 1) return;                       // single decoded tokens are another kernel's
    if (w.kv_begin & (P_BK - 1)) {
        if (threadIdx.x == 0) atomicOr(status, 32);
        return;
    }
    const int group = nh / nkv;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    const int kh = blockIdx.x / gparts;
    const int head0 = kh * group + (blockIdx.x % gparts) * heads_per_cta;
    const int n_heads = min(heads_per_cta, kh * group + group - head0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (w.kv_end - w.kv_begin + P_BK - 1) / P_BK;

    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t q_s = smem_u32(smem);
    const uint32_t kv_s = q_s + Q_BYTES;
    const uint32_t p_s = kv_s + P_STAGES * STAGE;
    unsigned char* ctl = smem + Q_BYTES + P_STAGES * STAGE + P_BYTES;
    const uint32_t bars = smem_u32(ctl);
    const uint32_t q_full = bars, kv_full = bars + 8, kv_empty = kv_full + 8 * P_STAGES, s_full = kv_empty + 8 * P_STAGES,
                   p_full = s_full + 16, p_empty = p_full + 8, o_full = p_empty + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctl + 8 * (2 * P_STAGES + 6));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ctl + 8 * (2 * P_STAGES + 6) + 8);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < P_STAGES; s++) { mbar_init(kv_full + 8 * s, 1); mbar_init(kv_empty + 8 * s, 1); }
        mbar_init(s_full, 1); mbar_init(s_full + 8, 1);
        mbar_init(p_full, 4);        // one arrival from each softmax warp
        mbar_init(p_empty, 1);
        mbar_init(o_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
        fence_async_smem();
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 4) {
        // ---- producer: the queries once, then key and value planes tile by tile --------------------
        pdl_wait();           // the queries and this step's cache rows come from the kernel before
        if (lane == 0) {
            mbar_expect_tx(q_full, (uint32_t)(NHALF * 128 * heads_per_cta * tile_tokens));
            for (int h = 0; h < NHALF; h++) tma_load_3d(q_s + h * P_ROWS * 128, &map_q, h * 64, head0, w.q_token0, q_full);
        }
        const int slab_rows = page_size < P_BK ? page_size : P_BK;
        const int slabs = P_BK / slab_rows;                  // at most 8
        const uint32_t slab_bytes = (uint32_t)slab_rows * 128;
        const int* table = block_tables + (size_t)w.seg * table_width;
        for (int t = 0; t < n_tiles; t++) {
            const int s = t % P_STAGES;
            const int kv0 = w.kv_begin + t * P_BK;
            if (t >= P_STAGES && !mbar_wait(kv_empty + 8 * s, ((t / P_STAGES) - 1) & 1, abort_flag)) break;
            // lane i looks up slab i's page
            int page = -1;
            if (lane < slabs) {
                const int j = kv0 + lane * slab_rows;
                if (j < w.kv_end && (j >> page_shift) < table_width) page = table[j >> page_shift];
                if (page >= n_pages) { atomicOr(status, 8); page = -1; }
            }
            const uint32_t have = __ballot_sync(0xffffffffu, page >= 0) & ((1u << slabs) - 1);
            const uint32_t st_base = kv_s + s * STAGE;
            unsigned char* st_ptr = smem + Q_BYTES + s * STAGE;
            if (have != (1u << slabs) - 1) {
                // slabs with no page behind them are zeroed by hand: nothing stale is multiplied
                for (int i = 0; i < slabs; i++) {
                    if (have & (1u << i)) continue;
                    for (int pl = 0; pl < 2 * NHALF; pl++)
                        for (int o = lane * 16; o < (int)slab_bytes; o += 32 * 16)
                            *reinterpret_cast<uint4*>(st_ptr + pl * P_PLANE + i * slab_bytes + o) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
                __syncwarp();
            }
            if (lane == 0) mbar_expect_tx(kv_full + 8 * s, 2 * NHALF * slab_bytes * __popc(have));
            __syncwarp();
            if (lane < slabs && page >= 0) {
                const int j = kv0 + lane * slab_rows;
                const int row = (page * nkv + kh) * page_size + (j & (page_size - 1));
                for (int h = 0; h < NHALF; h++) {
                    tma_load_2d(st_base + h * P_PLANE + lane * slab_bytes, &map_k, h * 64, row, kv_full + 8 * s);
                    tma_load_2d(st_base + (NHALF + h) * P_PLANE + lane * slab_bytes, &map_v, h * 64, row, kv_full + 8 * s);
                }
            }
        }
    } else if (warp == 5) {
        // ---- tensor-core issue ----------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(P_ROWS, P_BK), idesc_pv = instr_desc(P_ROWS, HD, 1);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            auto scores = [&](int t) {       // S[t & 1] = Q K_t^T
                const int s = t % P_STAGES;
                if (!mbar_wait(kv_full + 8 * s, (t / P_STAGES) & 1, abort_flag)) return false;
                tc_fence_after();
                const uint32_t k_base = kv_s + s * STAGE;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++)
                    mma_ss(tmem + S_COL + (t & 1) * P_BK, smem_desc(q_s + (ks / 4) * P_ROWS * 128 + (ks % 4) * 32),
                           smem_desc(k_base + (ks / 4) * P_PLANE + (ks % 4) * 32), idesc_qk, ks ? 1u : 0u);
                mma_commit(s_full + 8 * (t & 1));
                return true;
            };
            for (int t = 0; t < 2 && t < n_tiles && ok; t++) ok = scores(t);
            for (int t = 0; t < n_tiles && ok; t++) {
                if (!mbar_wait(p_full, t & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t v_base = kv_s + (t % P_STAGES) * STAGE + NHALF * P_PLANE;
#pragma unroll
                for (int ks = 0; ks < P_BK / 16; ks++)     // 16 keys = 2048 bytes down the value planes
                    mma_ss(tmem + O_COL, smem_desc(p_s + ks * 32), smem_desc(v_base + ks * 2048, P_PLANE), idesc_pv,
                           (t | ks) ? 1u : 0u);
                mma_commit(kv_empty + 8 * (t % P_STAGES));   // keys and values of this tile are read
                mma_commit(p_empty);                         // and so is P
                if (t + 2 < n_tiles) ok = scores(t + 2);
            }
            if (ok) mma_commit(o_full);
        }
    } else {
        // ---- softmax, one row a thread; then the epilogue -------------------------------------------
        pdl_launch_dependents();
        const int row = warp * 32 + lane;
        const int tq = row / heads_per_cta, hh = row % heads_per_cta;
        const bool live = tq < w.q_count && hh < n_heads && tq < tile_tokens;
        // keys below hi are visible to this row; rows that are no query's see everything (their
        // results are never stored, and a row of nothing but masked keys would make NaN)
        const int hi = live ? min(w.kv_end, w.q_pos0 + tq + 1) : w.kv_end;
        const uint32_t lane_base = tmem + ((uint32_t)(warp * 32) << 16);
        float m_used = -CUDART_INF_F, l_run = 0.f;
        bool ok = true;
#ifdef PLLM_ATTN_DEBUG
        const bool dbg = blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0;
        unsigned long long* stamps = reinterpret_cast<unsigned long long*>(part_o);
#define STAMP(k) if (dbg && t < 40) { unsigned long long ts; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ts)); stamps[t * 8 + (k)] = ts; }
#else
#define STAMP(k)
#endif
        for (int t = 0; t < n_tiles; t++) {
            const int kv0 = w.kv_begin + t * P_BK;
            STAMP(0)
            if (!mbar_wait(s_full + 8 * (t & 1), (t >> 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after();
            STAMP(1)
            uint32_t v0[32], v1[32];
            tmem_ld32(lane_base + S_COL + (t & 1) * P_BK, v0);
            tmem_ld32(lane_base + S_COL + (t & 1) * P_BK + 32, v1);
            tmem_wait_ld();
            // keys of this tile at or past vis are hidden from this row (only tiles on the diagonal have any)
            const int vis = hi - kv0;
            if (vis < P_BK) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (i >= vis) v0[i] = 0xff800000u;          // -inf
                    if (i + 32 >= vis) v1[i] = 0xff800000u;
                }
            }
            // the row's maximum, four chains side by side (one warp to a scheduler: the chain's latency is the time)
            float m4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
#pragma unroll
                for (int k = 0; k < 4; k++) m4[k] = fmaxf(m4[k], fmaxf(__uint_as_float(v0[i + k]), __uint_as_float(v1[i + k])));
            }
            const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale_log2;   // the scale is positive
            // move the maximum only when it grew by more than 2^8 (or is not set yet)
            const bool grow = mx > m_used + P_RESCALE || (m_used == -CUDART_INF_F && mx > -CUDART_INF_F);
            // P of the tile before this one must be read out of shared memory before it is overwritten,
            // and its O += P V done before O may be touched
            STAMP(2)
            if (t > 0 && !mbar_wait(p_empty, (t - 1) & 1, abort_flag)) { ok = false; break; }
            STAMP(3)
            if (t > 0 && __any_sync(0xffffffffu, grow)) {
                tc_fence_after();
                const float alpha = (grow && m_used > -CUDART_INF_F) ? ex2(m_used - mx) : (grow ? 0.f : 1.f);
                l_run *= alpha;
#pragma unroll
                for (int c = 0; c < HD / 32; c++) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + O_COL + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_base + O_COL + c * 32, o);
                }
                tmem_wait_st();
            }
            if (grow) m_used = mx;
            // weights 2^(s * scale - m): one multiply-add and one exponential each; a hidden key's -inf gives 0
            const float neg_m = m_used > -CUDART_INF_F ? -m_used : 0.f;
            uint32_t pw[32];
            float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const uint32_t a = i < 16 ? v0[2 * i] : v1[2 * i - 32], b2 = i < 16 ? v0[2 * i + 1] : v1[2 * i - 31];
                const float p0 = ex2(fmaf(__uint_as_float(a), scale_log2, neg_m));
                const float p1 = ex2(fmaf(__uint_as_float(b2), scale_log2, neg_m));
                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                pw[i] = *reinterpret_cast<uint32_t*>(&h);
                s4[i & 3] += p0 + p1;
            }
            const float sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
            l_run += sum;
            // the row's 128 bytes, chunk c at c ^ (row & 7)
            unsigned char* prow = smem + Q_BYTES + P_STAGES * STAGE + row * 128;
#pragma unroll
            for (int c = 0; c < 8; c++)
                *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pw[4 * c], pw[4 * c + 1], pw[4 * c + 2], pw[4 * c + 3]);
            STAMP(4)
            fence_async_smem();          // the tensor cores read shared memory through the async proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full);
            STAMP(5)
        }
        if (ok && mbar_wait(o_full, 0, abort_flag)) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
            for (int c = 0; c < HD / 32; c++) {
                uint32_t o[32];
                tmem_ld32(lane_base + O_COL + c * 32, o);
                tmem_wait_ld();
                if (!live) continue;
                const int head = head0 + hh;
                if (w.part_slot < 0) {
                    bf16* dst = out + ((size_t)(w.q_token0 + tq) * nh + head) * HD + c * 32;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        uint32_t pk[4];
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 2 * k]) * inv,
                                                                     __uint_as_float(o[8 * i + 2 * k + 1]) * inv);
                            pk[k] = *reinterpret_cast<uint32_t*>(&h);
                        }
                        *reinterpret_cast<uint4*>(dst + i * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                } else {
                    const size_t pr = (size_t)(w.part_slot + tq) * nh + head;
                    float* dst = part_o + pr * HD + c * 32;
#pragma unroll
                    for (int i = 0; i < 8; i++)
                        *reinterpret_cast<float4*>(dst + 4 * i) = make_float4(__uint_as_float(o[4 * i]), __uint_as_float(o[4 * i + 1]),
                                                                              __uint_as_float(o[4 * i + 2]), __uint_as_float(o[4 * i + 3]));
                    if (c == 0) { part_ml[pr * 2] = m_used * 0.6931471805599453f; part_ml[pr * 2 + 1] = l_run; }   // natural-log units
                }
            }
        }
    }
    // ---- everyone meets; the allocating warp gives the tensor memory back ---------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
    }
    if (threadIdx.x == 0 && *abort_flag) atomicOr(status, 128);
}

// The most query tokens an item of this kernel may hold.
PLLM_EXPORT int pllm_attention_prefill_tcgen05_tile_tokens(int nh, int nkv) {
    const int group = nh / nkv;
    const int heads_per_cta = group < 16 ? group : 16;
    return P_ROWS / heads_per_cta;
}

// Whether this kernel takes the several-token items of this shape and cache layout (swizzled rows).
PLLM_EXPORT int pllm_attention_prefill_tcgen05_supports(int dtype, int nh, int nkv, int hd, int page_size, int window) {
    return dtype == PLLM_BF16 && (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0 && window <= 0 && page_size >= 8 &&
           (page_size & (page_size - 1)) == 0;
}

template <int HD>
static int launch_prefill(const void* q, const void* k_pool, const void* v_pool, const int* block_tables, const int* work,
                          const int* n_work_ptr, int max_work, void* out, float* part_o, float* part_ml, int n_tokens,
                          int nh, int nkv, int page_size, int n_pages, int table_width, float scale, int* status,
                          cudaStream_t stream) {
    const int group = nh / nkv;
    const int heads_per_cta = group < 16 ? group : 16;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    const int tile_tokens = P_ROWS / heads_per_cta;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) page_shift++;
    const int slab_rows = page_size < P_BK ? page_size : P_BK;
    CUtensorMap map_q, map_k, map_v;
    {
        const long long dq[3] = {HD, nh, n_tokens}, sq[2] = {2LL * HD, 2LL * HD * nh};
        const int bq[3] = {64, heads_per_cta, tile_tokens};
        if (tensor_map(q, 3, dq, sq, bq, true, &map_q) != 0) return PLLM_ERR_SIZE;
        const long long dp[2] = {HD, (long long)n_pages * nkv * page_size}, sp[1] = {2LL * HD};
        const int bp[2] = {64, slab_rows};
        if (tensor_map(k_pool, 2, dp, sp, bp, false, &map_k) != 0) return PLLM_ERR_SIZE;
        if (tensor_map(v_pool, 2, dp, sp, bp, false, &map_v) != 0) return PLLM_ERR_SIZE;
    }
    constexpr int NHALF = HD / 64;
    const size_t smem = (size_t)NHALF * P_ROWS * 128 + (size_t)P_STAGES * 2 * NHALF * P_PLANE + P_ROWS * 128 +
                        8 * (2 * P_STAGES + 6) + 16 + 1024;
    cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(attention_prefill_tcgen05_kernel<HD>, dim3(nkv * gparts, max_work), dim3(P_THREADS), smem, stream, map_q,
                   map_k, map_v, block_tables, (const AttnWork*)work, n_work_ptr, (bf16*)out, part_o, part_ml, nh, nkv,
                   page_size, page_shift, n_pages, table_width, scale * 1.4426950408889634f, heads_per_cta, tile_tokens, status);
    return launch_status();
}

// q, out: [n_tokens, nh, hd] bfloat16; pools [n_pages, nkv, page_size, hd] with swizzled rows.
PLLM_EXPORT int pllm_attention_prefill_tcgen05(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                               const int* work, const int* n_work_ptr, int max_work, void* out,
                                               float* part_o, float* part_ml, int n_tokens, int nh, int nkv, int hd,
                                               int page_size, int n_pages, int table_width, float scale, int* status,
                                               cudaStream_t stream) {
    if (max_work <= 0 || n_tokens <= 0) return PLLM_OK;
    if (!pllm_attention_prefill_tcgen05_supports(PLLM_BF16, nh, nkv, hd, page_size, 0)) return PLLM_ERR_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return PLLM_ERR_ALIGN;
    if (hd == 128)
        return launch_prefill<128>(q, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, n_tokens,
                                   nh, nkv, page_size, n_pages, table_width, scale, status, stream);
    return launch_prefill<64>(q, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, n_tokens, nh,
                              nkv, page_size, n_pages, table_width, scale, status, stream);
}

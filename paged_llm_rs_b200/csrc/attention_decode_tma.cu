// Attention over the paged cache in bfloat16, head sizes 64 and 128, with the pages
// brought in by the bulk-copy engine: the serving kernel for decoding (one query
// token per request against its whole context, bound by the bytes of the keys and
// values) and for portions of prompts.  The reference's decode kernel
// (crates/pagedllm/src/kernels/paged_attention.cu:42-148) launches one block per
// (row, query head), re-reads every key once per query head of a group and keeps
// its scores in a buffer as long as the context; its prefill gathers the pages
// into a rectangle first (crates/pagedllm/src/model/attention.rs:190-214).  Here
// one CTA serves all query heads of a kv head from one copy of the keys, a long
// context is split over CTAs, nothing is gathered, and the softmax runs online.
//
// Pages come in with cp.async.bulk (the untiled TMA): a page's rows for one kv head
// are contiguous in the cache ([pages, kv_heads, page_size, head_dim]), so one
// elected thread moves a whole page slab (up to 64 rows) with one instruction and
// an mbarrier counts the bytes.  Nobody computes addresses per 16 bytes.  The
// cache stores each row's 16-byte chunks XOR-ed with the row's offset in its page
// (see qk_norm_rope_kv.cu), which is the layout ldmatrix wants in shared memory,
// so the slab is copied as it lies.
//
// A CTA has four consumer warps and one producer warp.  Tiles of 64 keys go round
// a 3-stage ring; every consumer warp reads every tile in turn (a parity wait tells
// two phases of a barrier apart and no more, so no warp may run a whole turn of the
// ring ahead of another: taking tiles in turn keeps them within it).  q.k^T and p.v
// run on mma.sync.m16n8k16.  For one query token the group's heads are the (padded)
// 16 rows of one block, each warp multiplies its own 16 keys of every tile and keeps
// a running (max, sum, output) of its own; the four meet in shared memory at the
// end.  For several query tokens the rows (token, head) are spread over the warps,
// 16 each, and every warp multiplies whole tiles.  Every wait on an mbarrier is
// bounded: a waiter that gives up raises a status bit, tells the others and the
// CTA returns.
//
// It takes items whose key range starts on a multiple of 64 and has no window, in
// caches whose pages hold a power of two of at least 8 tokens; the rest is the
// cp.async kernel's (attention_mma.cu).
#include "common.cuh"

#define TD_BK 64
#define TD_STAGES 3
#define TD_CONSUMERS 4
#define TD_QROWS 64      // query rows (token, head) a CTA may hold
#define TD_SPIN_LIMIT (1 << 18)

struct AttnWork { int seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split; };   // split: count << 16 | index

namespace {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits until the barrier's phase `parity` is over; gives up after a bounded number
// of polls or when another thread has given up.  Returns false then.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int spin = 0; spin < TD_SPIN_LIMIT; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// An 8x8 block of 16-bit values held one row in four lanes, transposed across the warp.
__device__ __forceinline__ uint32_t movmatrix_t(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
    return d;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <int HD> __device__ __forceinline__ uint32_t toff(int row, int chunk) {
    return (uint32_t)(row * (HD * 2) + ((chunk ^ (row & 7)) << 4));
}

}  // namespace

// What the kernel needs to do the work of the q/k norm + rotation + cache-write kernel itself, for
// steps of single decoded tokens (qkv null: not asked to).  The reference does these as separate
// tensor operations before its attention (crates/pagedllm/src/model/attention.rs:148-158); in a
// decode step each is a launch of a few microseconds for a few kilobytes.
struct FusedQK {
    const bf16* qkv;                 // [tokens, (nh + 2 nkv) * hd], the projection's output
    const float *q_gain, *k_gain;    // [hd] or null: no norm
    const float *cos_t, *sin_t;      // [max_pos, hd / 2] or null: no rotation
    bf16 *k_pool, *v_pool;           // the pools again, to write the token's own row
    float eps;
    int max_pos;
};

// One head's row, hd / 32 values a lane (lane l: dims l * VPL ..): the norm over the row, then the
// rotation of dim d with d +- hd / 2 (16 lanes away), in float; the arithmetic of qk_norm_rope_kv.cu.
template <int HD>
__device__ __forceinline__ void norm_rope_row(const bf16* src, const float* gain, const float* cs, const float* sn, float eps,
                                              int lane, float (&f)[HD / 32]) {
    constexpr int VPL = HD / 32;
#pragma unroll
    for (int k = 0; k < VPL; k++) f[k] = __bfloat162float(src[lane * VPL + k]);
    if (gain) {
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < VPL; k++) ss += f[k] * f[k];
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int k = 0; k < VPL; k++) f[k] = f[k] * inv * gain[lane * VPL + k];
    }
    if (cs) {
        const bool upper = lane >= 16;
#pragma unroll
        for (int k = 0; k < VPL; k++) {
            const float other = __shfl_xor_sync(0xffffffffu, f[k], 16);
            const int i = (lane & 15) * VPL + k;
            f[k] = upper ? f[k] * cs[i] + other * sn[i] : f[k] * cs[i] - other * sn[i];
        }
    }
}

template <int HD, bool KEYS_AS_ROWS>
__global__ void __launch_bounds__((TD_CONSUMERS + 1) * 32, 2) attention_decode_tma_kernel(
    const bf16* q, const bf16* k_pool, const bf16* v_pool,   // written by the kernels before this one: no __restrict__
    const int* __restrict__ block_tables, const AttnWork* __restrict__ work, const int* __restrict__ n_work_ptr,
    bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    int nh, int nkv, int page_size, int page_shift, int n_pages, int table_width, float scale_log2,
    int heads_per_cta, int kinds_mask, FusedQK fq, int* status) {
    // The work items and block tables came from the host before the step, and the cache below
    // the step's own positions was written by earlier steps: neither depends on the kernels
    // just before this one.  So nobody waits for those kernels yet: the producer starts the
    // first tiles of old keys on their way at once, and waits only before a tile that may hold
    // a key of this step; the consumers wait before they read the queries.
    if ((int)blockIdx.y >= *n_work_ptr) return;
    const AttnWork w = work[blockIdx.y];
    if (!(kinds_mask & (w.q_count == 1 ? 1 : 2))) return;   // another kernel's item
    if (KEYS_AS_ROWS && w.q_count != 1) return;             // (this variant is for single tokens only)
    if (w.kv_begin & (TD_BK - 1)) {
        // slabs and the swizzle need the range to start on a tile boundary
        if (threadIdx.x == 0) atomicOr(status, 32);
        return;
    }
    const int group = nh / nkv;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    const int kh = blockIdx.x / gparts;
    const int head0 = kh * group + (blockIdx.x % gparts) * heads_per_cta;
    const int n_heads = min(heads_per_cta, kh * group + group - head0);
    const int rows = w.q_count * n_heads;          // <= 64: (token, head) pairs
    const bool decode = w.q_count == 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int KSTEPS = HD / 16, DTILES = HD / 8, CH = HD / 8;
    constexpr int TILE_BYTES = TD_BK * HD * 2;          // keys (or values) of one tile
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;

    extern __shared__ __align__(128) unsigned char smem[];
    const uint32_t base = smem_u32(smem);
    const uint32_t q_s = base + TD_STAGES * STAGE_BYTES;
    const uint32_t bars = q_s + TD_QROWS * HD * 2;       // full[S], empty[S]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + TD_STAGES * STAGE_BYTES + TD_QROWS * HD * 2 + 16 * TD_STAGES);

    if (threadIdx.x == 0) {
        for (int s = 0; s < TD_STAGES; s++) {
            mbar_init(bars + 8 * s, 1);                      // full: the producer's arrive, plus the bytes
            mbar_init(bars + 8 * (TD_STAGES + s), TD_CONSUMERS);   // empty: every consumer warp's release
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
        asm volatile("fence.proxy.async.shared::cta;\n" ::);
    }
    __syncthreads();   // the barriers are set up; the producer goes its own way from here

    const int n_tiles = (w.kv_end - w.kv_begin + TD_BK - 1) / TD_BK;
    const int slab_rows = page_size < TD_BK ? page_size : TD_BK;
    const int slabs = TD_BK / slab_rows;          // at most 8 (pages of at least 8 tokens)
    const uint32_t slab_bytes = (uint32_t)slab_rows * HD * 2;

    if (warp == TD_CONSUMERS) {
        // ---- producer: page slabs into the ring ---------------------------------------------
        const int* table = block_tables + (size_t)w.seg * table_width;
        // the table entries of the key range, 32 at a time, one in each lane: no tile waits for a lookup
        int win0 = w.kv_begin >> page_shift;
        int tbl = (win0 + lane < table_width) ? table[win0 + lane] : -1;
        bool waited = false;
        for (int t = 0; t < n_tiles; t++) {
            const int s = t % TD_STAGES;
            const int kv0 = w.kv_begin + t * TD_BK;
            // A decoded token's own key is the only one this step writes for its request; a
            // portion's tiles read keys that other tiles of the portion bring, so they wait first.
            if (!waited && (!decode || kv0 + TD_BK > w.q_pos0)) { pdl_wait(); waited = true; }
            if (((kv0 + TD_BK - 1) >> page_shift) >= win0 + 32) {
                win0 = kv0 >> page_shift;
                tbl = (win0 + lane < table_width) ? table[win0 + lane] : -1;
            }
            if (t >= TD_STAGES && !mbar_wait(bars + 8 * (TD_STAGES + s), ((t / TD_STAGES) - 1) & 1, abort_flag)) break;
            const uint32_t k_dst = base + s * STAGE_BYTES, v_dst = k_dst + TILE_BYTES;
            // which slabs exist: a page of the table at or before the range's last key
            uint32_t have = 0;
            int pg[8];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                pg[i] = -1;
                if (i >= slabs) continue;
                const int j = kv0 + i * slab_rows;
                int page = __shfl_sync(0xffffffffu, tbl, ((j >> page_shift) - win0) & 31);
                if (j >= w.kv_end) page = -1;
                if (page >= n_pages) { if (lane == 0) atomicOr(status, 8); page = -1; }
                pg[i] = page;
                if (page >= 0) have |= 1u << i;
            }
            // slabs with no page behind them are zeroed by hand: nothing stale or unset is multiplied
            if (have != (1u << slabs) - 1) {
                for (int i = 0; i < slabs; i++) {
                    if (have & (1u << i)) continue;
                    for (int o = lane * 16; o < (int)slab_bytes; o += 32 * 16) {
                        *reinterpret_cast<uint4*>(smem + s * STAGE_BYTES + i * slab_bytes + o) = make_uint4(0, 0, 0, 0);
                        *reinterpret_cast<uint4*>(smem + s * STAGE_BYTES + TILE_BYTES + i * slab_bytes + o) = make_uint4(0, 0, 0, 0);
                    }
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // the zeros before the copies
                __syncwarp();
            }
            if (lane == 0) {
                mbar_expect_tx(bars + 8 * s, 2 * slab_bytes * __popc(have));
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    if (i >= slabs || pg[i] < 0) continue;
                    const int j = kv0 + i * slab_rows;
                    const size_t src = (((size_t)pg[i] * nkv + kh) * page_size + (j & (page_size - 1))) * HD;
                    bulk_copy(k_dst + i * slab_bytes, k_pool + src, slab_bytes, bars + 8 * s);
                    bulk_copy(v_dst + i * slab_bytes, v_pool + src, slab_bytes, bars + 8 * s);
                }
            }
        }
        return;
    }

    // the query rows, zero beyond them (the first tiles are on their way meanwhile)
    const bool fused = fq.qkv != nullptr && decode;
    // fused: this CTA's range ends with the token's own key, which it makes itself (norm, rotation),
    // stores to the cache for later steps and puts into the last tile in shared memory
    const bool owns_new = fused && w.kv_end == w.q_pos0 + 1 && w.kv_end > w.kv_begin;   // (not an empty item that ends there)
    constexpr int VPL = HD / 32;
    uint32_t new_k[VPL / 2], new_v[VPL / 2];       // the row's values of this lane, packed (warps 2 and 3)
    if (fused) {
        int pos = w.q_pos0;
        if (fq.cos_t && (pos < 0 || pos >= fq.max_pos)) { if (threadIdx.x == 0) atomicOr(status, 4); pos = 0; }
        const float* cs = fq.cos_t ? fq.cos_t + (size_t)pos * (HD / 2) : nullptr;
        const float* sn = fq.sin_t ? fq.sin_t + (size_t)pos * (HD / 2) : nullptr;
        const int heads_total = nh + 2 * nkv;
        pdl_wait(KID_ATT_TMA);
        const bf16* tok = fq.qkv + (size_t)w.q_token0 * heads_total * HD;
        for (int row = warp; row < 16; row += TD_CONSUMERS) {
            uint32_t pk[VPL / 2];
#pragma unroll
            for (int k = 0; k < VPL / 2; k++) pk[k] = 0;
            if (row < n_heads) {
                float f[VPL];
                norm_rope_row<HD>(tok + (size_t)(head0 + row) * HD, fq.q_gain, cs, sn, fq.eps, lane, f);
#pragma unroll
                for (int k = 0; k < VPL / 2; k++) pk[k] = pack2(f[2 * k], f[2 * k + 1]);
            }
            // lane l's values are dims l * VPL ..: chunk (l * VPL) / 8 of the row, (l * VPL) % 8 values in
            unsigned char* dst = smem + TD_STAGES * STAGE_BYTES + toff<HD>(row, lane * VPL / 8) + (lane * VPL % 8) * 2;
#pragma unroll
            for (int k = 0; k < VPL / 2; k++) reinterpret_cast<uint32_t*>(dst)[k] = pk[k];
        }
        if (owns_new && warp >= TD_CONSUMERS - 2) {
            const bool is_k = warp == TD_CONSUMERS - 2;
            float f[VPL];
            norm_rope_row<HD>(tok + (size_t)(nh + (is_k ? 0 : nkv) + kh) * HD, is_k ? fq.k_gain : nullptr, is_k ? cs : nullptr,
                              is_k ? sn : nullptr, fq.eps, lane, f);
            uint32_t pk[VPL / 2];
#pragma unroll
            for (int k = 0; k < VPL / 2; k++) pk[k] = pack2(f[2 * k], f[2 * k + 1]);
            // into the cache, chunk c at c ^ (offset in page & 7), for the steps to come
            const int page = block_tables[(size_t)w.seg * table_width + (w.q_pos0 >> page_shift)];
            const int off = w.q_pos0 & (page_size - 1);
            if (page >= 0 && page < n_pages) {
                bf16* row_w = (is_k ? fq.k_pool : fq.v_pool) + (((size_t)page * nkv + kh) * page_size + off) * HD;
                uint32_t* dst = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(row_w) +
                                                            (((lane * VPL / 8) ^ (off & 7)) << 4) + (lane * VPL % 8) * 2);
#pragma unroll
                for (int k = 0; k < VPL / 2; k++) dst[k] = pk[k];
            } else if (lane == 0) {
                atomicOr(status, 2);
            }
#pragma unroll
            for (int k = 0; k < VPL / 2; k++) { if (is_k) new_k[k] = pk[k]; else new_v[k] = pk[k]; }
        }
    } else {
        pdl_wait(KID_ATT_TMA);
        for (int idx = threadIdx.x; idx < (decode ? 16 : TD_QROWS) * CH; idx += TD_CONSUMERS * 32) {
            const int row = idx / CH, chunk = idx % CH;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (row < rows)
                v = *reinterpret_cast<const uint4*>(q + ((size_t)(w.q_token0 + row / n_heads) * nh + head0 + row % n_heads) * HD + chunk * 8);
            *reinterpret_cast<uint4*>(smem + TD_STAGES * STAGE_BYTES + toff<HD>(row, chunk)) = v;
        }
    }
    asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));

    float* o_s = reinterpret_cast<float*>(smem);          // [4][16][HD], once the ring is no longer read
    float* ml_s = o_s + TD_CONSUMERS * 16 * HD;           // [4][16][2]
    if constexpr (KEYS_AS_ROWS) {
    // ---- consumers, one query token of at most 8 heads: the KEYS are the 16 rows of the score block --------
    // and the heads its 8 columns, S^T = K q^T and O^T = V^T P^T.  A block of 16 keys costs 8 + HD / 16
    // mma instead of twice that with the (two, four, eight) heads padded to 16 rows, the output is
    // HD / 16 x 4 registers instead of HD / 8 x 4, and the queries are 2 registers a k-step instead of 4.
    uint32_t qb[KSTEPS][2];
    {
#pragma unroll
        for (int kp = 0; kp < KSTEPS / 2; kp++) {
            uint32_t r[4];
            ldsm4(r, q_s + toff<HD>(lane & 7, kp * 4 + (lane >> 3)));
            qb[2 * kp][0] = r[0]; qb[2 * kp][1] = r[1]; qb[2 * kp + 1][0] = r[2]; qb[2 * kp + 1][1] = r[3];
        }
    }
    const int hi0 = min(w.kv_end, w.q_pos0 + 1);     // keys the token may see, the same for all its heads
    // this thread: keys lane / 4 and + 8 of the warp's 16, heads 2 * (lane % 4) and + 1
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
    constexpr int MT = HD / 16;
    float o_acc[MT][4];
#pragma unroll
    for (int d = 0; d < MT; d++) { o_acc[d][0] = o_acc[d][1] = o_acc[d][2] = o_acc[d][3] = 0.f; }
    const int key_base = warp * 16;
    const int mat = lane >> 3;
    for (int t = 0; t < n_tiles; t++) {
        const int s = t % TD_STAGES;
        if (!mbar_wait(bars + 8 * s, (t / TD_STAGES) & 1, abort_flag)) break;
        const int kv0 = w.kv_begin + t * TD_BK + key_base;
        const uint32_t k_s = base + s * STAGE_BYTES, v_s = k_s + TILE_BYTES;
        if (owns_new && t == n_tiles - 1) {
            // the token's own key and value over what the copy brought for that row (whatever the page held)
            if (warp >= TD_CONSUMERS - 2) {
                const int r = w.q_pos0 - (w.kv_begin + t * TD_BK);
                unsigned char* dst = smem + s * STAGE_BYTES + (warp == TD_CONSUMERS - 2 ? 0 : TILE_BYTES) +
                                     toff<HD>(r, lane * VPL / 8) + (lane * VPL % 8) * 2;
#pragma unroll
                for (int k = 0; k < VPL / 2; k++)
                    reinterpret_cast<uint32_t*>(dst)[k] = warp == TD_CONSUMERS - 2 ? new_k[k] : new_v[k];
            }
            asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
        }
        if (kv0 < hi0) {
            // the warp's 16 keys and values into registers, and the stage goes back to the producer
            // before the arithmetic: the next copy into it is on its way while this one is multiplied
            const int krow = key_base + (lane & 7) + (mat & 1) * 8;
            const int vkey = key_base + (lane & 7) + (mat >> 1) * 8;
            uint32_t kf[KSTEPS][4], vf[MT][4];
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks++) ldsm4(kf[ks], k_s + toff<HD>(krow, ks * 2 + (mat >> 1)));
#pragma unroll
            for (int d = 0; d < MT; d++) ldsm4_t(vf[d], v_s + toff<HD>(vkey, d * 2 + (mat & 1)));
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + 8 * (TD_STAGES + s));
            // two chains of mma over the k-steps, added at the end
            float sa[4] = {0.f, 0.f, 0.f, 0.f}, sb[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < KSTEPS; ks += 2) {
                mma(sa, kf[ks], qb[ks][0], qb[ks][1]);
                mma(sb, kf[ks + 1], qb[ks + 1][0], qb[ks + 1][1]);
            }
            const int j0 = kv0 + (lane >> 2);
            const bool see0 = j0 < hi0, see1 = j0 + 8 < hi0;
            float sc[4];
            sc[0] = see0 ? (sa[0] + sb[0]) * scale_log2 : -CUDART_INF_F;
            sc[1] = see0 ? (sa[1] + sb[1]) * scale_log2 : -CUDART_INF_F;
            sc[2] = see1 ? (sa[2] + sb[2]) * scale_log2 : -CUDART_INF_F;
            sc[3] = see1 ? (sa[3] + sb[3]) * scale_log2 : -CUDART_INF_F;
            float mx[2] = {fmaxf(sc[0], sc[2]), fmaxf(sc[1], sc[3])};
            float corr[2], m_use[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 4));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 8));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 16));
                const float m_new = fmaxf(m_run[i], mx[i]);
                m_use[i] = m_new == -CUDART_INF_F ? 0.f : m_new;
                corr[i] = exp2f(m_run[i] - m_use[i]);
                m_run[i] = m_new;
                l_run[i] *= corr[i];
            }
            const float p0 = exp2f(sc[0] - m_use[0]), p1 = exp2f(sc[1] - m_use[1]);
            const float p2 = exp2f(sc[2] - m_use[0]), p3 = exp2f(sc[3] - m_use[1]);
            l_run[0] += p0 + p2;
            l_run[1] += p1 + p3;
            // P^T as the second operand: (key, head pair) in this thread becomes (head, key pair)
            const uint32_t pb0 = movmatrix_t(pack2(p0, p1)), pb1 = movmatrix_t(pack2(p2, p3));
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
                for (int d = 0; d < MT; d++) {
                    o_acc[d][0] *= corr[0]; o_acc[d][1] *= corr[1];
                    o_acc[d][2] *= corr[0]; o_acc[d][3] *= corr[1];
                }
            }
#pragma unroll
            for (int d = 0; d < MT; d++) mma(o_acc[d], vf[d], pb0, pb1);
        } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(bars + 8 * (TD_STAGES + s));
        }
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 4);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 8);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 16);
    }
    pdl_launch_dependents();   // the key tiles are done: the next kernel's CTAs may take their places
    asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
    if (*abort_flag) {
        if (threadIdx.x == 0) atomicOr(status, 16);
        return;
    }
    // the four warps' results meet, head by head
    {
        const int qh = (lane & 3) * 2;
#pragma unroll
        for (int d = 0; d < MT; d++) {
            float* a = o_s + ((size_t)(warp * 16 + qh) * HD + d * 16 + (lane >> 2));
            a[0] = o_acc[d][0]; a[HD] = o_acc[d][1];
            a[8] = o_acc[d][2]; a[HD + 8] = o_acc[d][3];
        }
        if (lane < 4) {
            ml_s[(warp * 16 + qh) * 2] = m_run[0]; ml_s[(warp * 16 + qh) * 2 + 1] = l_run[0];
            ml_s[(warp * 16 + qh + 1) * 2] = m_run[1]; ml_s[(warp * 16 + qh + 1) * 2 + 1] = l_run[1];
        }
    }
    } else {
    // ---- consumers ------------------------------------------------------------------------------
    // One query token: the group's heads are ONE 16-row block and the warps share each tile's
    // keys (16 each).  Several query tokens: the rows (token, head) are spread over the warps,
    // 16 each, and every warp multiplies all 64 keys of a tile.
    const int rbase = decode ? 0 : warp * 16;
    uint32_t qf[KSTEPS][4];
    {
        const int mat = lane >> 3;
        const int row = rbase + (lane & 7) + (mat & 1) * 8;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) ldsm4(qf[ks], q_s + toff<HD>(row, ks * 2 + (mat >> 1)));
    }
    // the two rows of this thread and the keys they may see
    const int r0 = rbase + (lane >> 2), r1 = r0 + 8;
    int hi[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int r = i ? r1 : r0;
        hi[i] = r < rows ? min(w.kv_end, w.q_pos0 + r / n_heads + 1) : 0;
    }
    int warp_hi = max(hi[0], hi[1]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) warp_hi = max(warp_hi, __shfl_xor_sync(0xffffffffu, warp_hi, o));
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
    float o_acc[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; d++) { o_acc[d][0] = o_acc[d][1] = o_acc[d][2] = o_acc[d][3] = 0.f; }
    bool alive = true;

    const int key_base = decode ? warp * (TD_BK / TD_CONSUMERS) : 0;
    const int np_count = decode ? TD_BK / TD_CONSUMERS / 16 : TD_BK / 16;   // pairs of 8-key score tiles: 1 or 4
    for (int t = 0; t < n_tiles && alive; t++) {
        const int s = t % TD_STAGES;
        if (!mbar_wait(bars + 8 * s, (t / TD_STAGES) & 1, abort_flag)) { alive = false; break; }
        const int kv0 = w.kv_begin + t * TD_BK + key_base;
        const uint32_t k_s = base + s * STAGE_BYTES, v_s = k_s + TILE_BYTES;
        if (owns_new && t == n_tiles - 1) {
            // the token's own key and value over what the copy brought for that row (whatever the page held)
            if (warp >= TD_CONSUMERS - 2) {
                const int r = w.q_pos0 - (w.kv_begin + t * TD_BK);
                unsigned char* dst = smem + s * STAGE_BYTES + (warp == TD_CONSUMERS - 2 ? 0 : TILE_BYTES) +
                                     toff<HD>(r, lane * VPL / 8) + (lane * VPL % 8) * 2;
#pragma unroll
                for (int k = 0; k < VPL / 2; k++)
                    reinterpret_cast<uint32_t*>(dst)[k] = warp == TD_CONSUMERS - 2 ? new_k[k] : new_v[k];
            }
            asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
        }
        if (kv0 < warp_hi) {   // some key of this warp's share is visible to one of its rows
            float s_acc[8][4];
#pragma unroll
            for (int n = 0; n < 8; n++) { s_acc[n][0] = s_acc[n][1] = s_acc[n][2] = s_acc[n][3] = 0.f; }
            {
                // one k-step at a time over all key tiles: neighbouring mma write different accumulators
                const int mat = lane >> 3;
                const int key0 = key_base + (lane & 7) + (mat >> 1) * 8;
#pragma unroll
                for (int ks = 0; ks < KSTEPS; ks++) {
                    uint32_t kf[4][4];
#pragma unroll
                    for (int np = 0; np < 4; np++)
                        if (np < np_count) ldsm4(kf[np], k_s + toff<HD>(key0 + np * 16, ks * 2 + (mat & 1)));
#pragma unroll
                    for (int np = 0; np < 4; np++) {
                        if (np >= np_count) break;
                        mma(s_acc[np * 2], qf[ks], kf[np][0], kf[np][1]);
                        mma(s_acc[np * 2 + 1], qf[ks], kf[np][2], kf[np][3]);
                    }
                }
            }
            float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
            const bool whole = kv0 + np_count * 16 <= min(hi[0], hi[1]);   // every key visible to both rows
#pragma unroll
            for (int n = 0; n < 8; n++) {
                if (n >= np_count * 2) break;
                const int j = kv0 + n * 8 + (lane & 3) * 2;
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float v = (whole || j + (e & 1) < hi[e >> 1]) ? s_acc[n][e] * scale_log2 : -CUDART_INF_F;
                    s_acc[n][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            }
            float corr[2], m_use[2];
#pragma unroll
            for (int i = 0; i < 2; i++) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m_run[i], mx[i]);
                m_use[i] = m_new == -CUDART_INF_F ? 0.f : m_new;
                corr[i] = exp2f(m_run[i] - m_use[i]);
                m_run[i] = m_new;
                l_run[i] *= corr[i];
            }
            uint32_t pf[4][4];
#pragma unroll
            for (int n = 0; n < 8; n++) {
                if (n >= np_count * 2) break;
                const float p0 = exp2f(s_acc[n][0] - m_use[0]), p1 = exp2f(s_acc[n][1] - m_use[0]);
                const float p2 = exp2f(s_acc[n][2] - m_use[1]), p3 = exp2f(s_acc[n][3] - m_use[1]);
                l_run[0] += p0 + p1;
                l_run[1] += p2 + p3;
                pf[n >> 1][(n & 1) * 2] = pack2(p0, p1);
                pf[n >> 1][(n & 1) * 2 + 1] = pack2(p2, p3);
            }
            // the running maximum seldom moves after the first tiles: rescale only when it did
            if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
                for (int d = 0; d < DTILES; d++) {
                    o_acc[d][0] *= corr[0]; o_acc[d][1] *= corr[0];
                    o_acc[d][2] *= corr[1]; o_acc[d][3] *= corr[1];
                }
            }
            {
                const int mat = lane >> 3;
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
                    if (kk >= np_count) break;
                    const int key = key_base + kk * 16 + (lane & 7) + (mat & 1) * 8;
                    // four fragment loads in flight, then their eight mma
#pragma unroll
                    for (int d4 = 0; d4 < DTILES / 2; d4 += 4) {
                        uint32_t vf[4][4];
#pragma unroll
                        for (int i = 0; i < 4; i++) ldsm4_t(vf[i], v_s + toff<HD>(key, (d4 + i) * 2 + (mat >> 1)));
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            mma(o_acc[(d4 + i) * 2], pf[kk], vf[i][0], vf[i][1]);
                            mma(o_acc[(d4 + i) * 2 + 1], pf[kk], vf[i][2], vf[i][3]);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + 8 * (TD_STAGES + s));   // this warp is done with the stage
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }
    pdl_launch_dependents();   // the key tiles are done: the next kernel's CTAs may take their places
    // (named barriers from here on: the producer warp has left)
    asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
    if (*abort_flag) {   // set before the warp that gave up reached the barrier: all see it alike
        if (threadIdx.x == 0) atomicOr(status, 16);
        return;
    }
    if (!decode) {
        // ---- several query tokens: every warp owns its rows' results ----------------------------
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
                    *reinterpret_cast<uint32_t*>(o + d * 8) = pack2(o_acc[d][i * 2] * inv, o_acc[d][i * 2 + 1] * inv);
            } else {
                const size_t pr = (size_t)(w.part_slot + tq) * nh + head;
                float* o = part_o + pr * HD + (lane & 3) * 2;
#pragma unroll
                for (int d = 0; d < DTILES; d++) { o[d * 8] = o_acc[d][i * 2]; o[d * 8 + 1] = o_acc[d][i * 2 + 1]; }
                if ((lane & 3) == 0) { part_ml[pr * 2] = m_run[i] * 0.6931471805599453f; part_ml[pr * 2 + 1] = l_run[i]; }
            }
        }
    } else {
    // ---- one query token: the four warps' results meet ---------------------------------------
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
    }
    }
    if (decode) {
    asm volatile("bar.sync 1, %0;\n" ::"n"(TD_CONSUMERS * 32));
    for (int idx = threadIdx.x; idx < rows * HD; idx += TD_CONSUMERS * 32) {
        const int r = idx / HD, c = idx % HD;
        float M = -CUDART_INF_F;
#pragma unroll
        for (int wi = 0; wi < TD_CONSUMERS; wi++) M = fmaxf(M, ml_s[(wi * 16 + r) * 2]);
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int wi = 0; wi < TD_CONSUMERS; wi++) {
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
            if (c == 0) { part_ml[pr * 2] = M * 0.6931471805599453f; part_ml[pr * 2 + 1] = L; }   // natural-log units
        }
    }
    }

}

// Whether this kernel takes decode items of this shape and cache layout.
PLLM_EXPORT int pllm_attention_decode_tma_supports(int dtype, int nh, int nkv, int hd, int page_size, int window) {
    return dtype == PLLM_BF16 && (hd == 64 || hd == 128) && nkv > 0 && nh % nkv == 0 && window <= 0 && page_size >= 8 &&
           (page_size & (page_size - 1)) == 0;
}

template <int HD>
static int launch_tma(const void* q, const void* k_pool, const void* v_pool, const int* block_tables, const int* work,
                      const int* n_work_ptr, int max_work, void* out, float* part_o, float* part_ml, int nh, int nkv,
                      int page_size, int n_pages, int table_width, float scale, int kinds_mask,
                      FusedQK fq, int* status, cudaStream_t stream) {
    const int group = nh / nkv;
    const int heads_per_cta = group < 16 ? group : 16;
    const int gparts = (group + heads_per_cta - 1) / heads_per_cta;
    int page_shift = 0;
    while ((1 << page_shift) < page_size) page_shift++;
    const size_t smem = (size_t)TD_STAGES * 2 * TD_BK * HD * 2 + TD_QROWS * HD * 2 + 16 * TD_STAGES + 16;
    const float scale_log2 = scale * 1.4426950408889634f;
    const dim3 block((TD_CONSUMERS + 1) * 32);
    // single tokens of groups of at most 8 heads go to the variant with the keys as rows; what else the
    // caller asked for (several query tokens) to the other, as a launch of its own
    int rest = kinds_mask;
    if (group <= 8 && (kinds_mask & 1)) {
        cudaFuncSetAttribute(attention_decode_tma_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_chained(attention_decode_tma_kernel<HD, true>, dim3(nkv * gparts, max_work), block, smem,
                       stream, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_tables, (const AttnWork*)work,
                       n_work_ptr, (bf16*)out, part_o, part_ml, nh, nkv, page_size, page_shift, n_pages, table_width,
                       scale_log2, heads_per_cta, 1, fq, status);
        rest &= ~1;
    }
    if (rest) {
        cudaFuncSetAttribute(attention_decode_tma_kernel<HD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        launch_chained(attention_decode_tma_kernel<HD, false>, dim3(nkv * gparts, max_work), block, smem,
                       stream, (const bf16*)q, (const bf16*)k_pool, (const bf16*)v_pool, block_tables, (const AttnWork*)work,
                       n_work_ptr, (bf16*)out, part_o, part_ml, nh, nkv, page_size, page_shift, n_pages, table_width,
                       scale_log2, heads_per_cta, rest, fq, status);
    }
    return launch_status();
}

static int dispatch_tma(const void* q, const void* k_pool, const void* v_pool, const int* block_tables, const int* work,
                        const int* n_work_ptr, int max_work, void* out, float* part_o, float* part_ml, int nh, int nkv,
                        int hd, int page_size, int n_pages, int table_width, float scale, int kinds_mask,
                        FusedQK fq, int* status, cudaStream_t stream) {
    if (max_work <= 0) return PLLM_OK;
    if (!pllm_attention_decode_tma_supports(PLLM_BF16, nh, nkv, hd, page_size, 0)) return PLLM_ERR_SIZE;
    if (hd == 128)
        return launch_tma<128>(q, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, nh, nkv,
                               page_size, n_pages, table_width, scale, kinds_mask, fq, status, stream);
    return launch_tma<64>(q, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, nh, nkv,
                          page_size, n_pages, table_width, scale, kinds_mask, fq, status, stream);
}

PLLM_EXPORT int pllm_attention_decode_tma(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                          const int* work, const int* n_work_ptr, int max_work, void* out,
                                          float* part_o, float* part_ml, int nh, int nkv, int hd, int page_size,
                                          int n_pages, int table_width, float scale, int kinds_mask, int* status,
                                          cudaStream_t stream) {
    FusedQK none = {};
    return dispatch_tma(q, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, nh, nkv, hd,
                        page_size, n_pages, table_width, scale, kinds_mask, none, status, stream);
}

// The same for a step of single decoded tokens, straight from the projection's output: the kernel
// norms and rotates the queries and each token's new key itself and writes key and value to the
// cache (rotation over the whole head or none; gains and tables may be null).
PLLM_EXPORT int pllm_attention_decode_tma_fused(const void* qkv, const float* q_gain, const float* k_gain, float eps,
                                                const float* cos_t, const float* sin_t, int max_pos, void* k_pool,
                                                void* v_pool, const int* block_tables, const int* work,
                                                const int* n_work_ptr, int max_work, void* out, float* part_o,
                                                float* part_ml, int nh, int nkv, int hd, int page_size, int n_pages,
                                                int table_width, float scale, int* status, cudaStream_t stream) {
    if (qkv == nullptr || ((uintptr_t)qkv & 15)) return PLLM_ERR_ALIGN;
    FusedQK fq = {(const bf16*)qkv, q_gain, k_gain, cos_t, sin_t, (bf16*)k_pool, (bf16*)v_pool, eps, max_pos};
    return dispatch_tma(nullptr, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, nh, nkv, hd,
                        page_size, n_pages, table_width, scale, 1, fq, status, stream);
}

PLLM_TRACE_EXPORT(attention_decode_tma)

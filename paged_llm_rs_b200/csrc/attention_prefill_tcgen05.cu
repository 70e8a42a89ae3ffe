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
//                 P rounded to bfloat16 back into tensor memory (tcgen05.st, two weights a column,
//                 over the first half of the scores they came from)
//   O += P V      tcgen05.mma with P as its tensor-memory operand and the value tile in shared
//                 memory, 128 x head_dim; a group's O stays in tensor memory for the whole item
//
// Sixteen warps: 0-3 and 4-7 are two softmax groups that take the key tiles in turn (even tiles
// the first, odd the second: a group's warp w owns rows 32 w .. 32 w + 31), 8 and 10 are the producers
// of the even tiles (TMA: queries and key tiles; value tiles), 12 and 13 those of the odd tiles.  Each
// group has two issuing threads of its own: one lane of warp 9 (14 for the second group) issues the
// tcgen05.mma of its scores, one of warp 11 (15) those of its sums; warp 9 also allocates the tensor
// memory.  The softmax warps take 192 registers a thread and leave the others 64 (setmaxnreg).
// Each group has a maximum, a sum and an O of its own for its half of the tiles (like two splits of the
// key range): nothing passes between the groups tile by tile, and they meet once, in the epilogue.  A
// row's running maximum is only moved when it grew by more than 2^8 (then the group's O is rescaled in
// tensor memory), which is exact after the final division.
// Tensor memory: two buffers of scores a group (4 x 64 columns), then head_dim columns of O a group
// (512 columns at head_dim 128).  A buffer takes the scores of the group's tile after next once the
// products that read this tile's weights out of it are over, so a tile's scores are formed while the
// group is busy with the tile before.
// The two groups share one unit for the exponentials, and left alone they fall into step: both compute
// their exponentials at once, at half speed each, and then both load, store and wait at once (started
// half a turn apart they were in step again within forty tiles).  So the exponentials take turns: a group
// begins its tile's when the other is through with those of the tile before (a barrier a group).
//
// What was measured on the way (16 heads over 8 kv heads of 128; one CTA's clocks a tile of 64 keys;
// -DPLLM_ATT_CLOCKS=1 builds the counters and a table of who saw what when).  A request to the copy engine
// costs the issuing warp 110-160 clocks whatever it moves, and 277 when one lane issues them one after the
// other: so a page is one request, the lanes of a warp issue a tile's pages in one instruction, and two
// warps share a ring (the loads alone then take 430 clocks a tile, 780 with one warp a ring).  A
// tcgen05.mma or a commit costs its lone thread some 85 clocks and a wait on a barrier that is long over
// 100-200 beside eight busy warps, so a thread waits first for what is surely there.  The 64 exponentials
// of a row's tile take a warp alone on its scheduler 704 clocks (512 would be the unit's rate), 1083 with
// the sums formed pairwise first, and two warps on one scheduler 1127 each.
// 8192 tokens: 295.6 us with one issuing thread for the scores of both groups (two tiles to one set of
// products) and one for the sums, the groups in step, a tile every 1250 clocks; 268.8 with issuing threads
// a group and the exponentials by turns; 255.1 (1077 TFLOP/s) with the scores buffered twice.  2048 tokens:
// 28.7 -> 26.1 us with the reduction's launch.  What bounds it now is the chain from a tile's weights to
// the scores of the tile after next (a wake-up, four products and a commit, a wake-up, eight products and
// a commit, a wake-up: some 2450 clocks).  A buffer's next scores wait for that chain and the chain for the
// group's turn on the buffer's tile (1750 clocks from the scores to the weights), so two of a group's tiles
// take turn + chain = 4200 clocks, a tile of the CTA 1050: what shortens either by x gains x / 4 a tile
// (without the maximum the 8192 tokens take 246 us, with half of the exponentials 251).
// Tried and no faster: three groups; rings of 2, 3 or 6 tiles; Q in tensor memory; polling with test_wait
// or with a time to stay suspended (319); the issuing loops run by their whole warps with an elected lane;
// one issuing thread a group for scores and sums (293); four issuing threads, each issuing a tile's sums
// and then the scores of the tile after next without a wait in between (283); turns of 128 keys with the
// weights through shared memory and the scores buffered once (276: the exponentials then take 19 clocks
// each instead of 14); two buffers of scores AND of weights with one O and the pair's maximum exchanged
// between twin warps (2700 clocks a pair); a part of the exponentials as a polynomial on the multiply-add
// units (a quarter: 929 clocks for the 64 against 704).
//
// Shared-memory layouts.  A tile for the tensor cores has rows of 128 bytes (64 values) with
// the 128-byte swizzle (tcgen05.cuh), in groups of 8 rows (1024 bytes).  The cache stores a key's
// or value's row (head_dim values) with its 16-byte chunk c at c ^ (offset in page & 7), which
// within each half of 64 values IS that swizzle.  A page's rows of one kv head are fetched by ONE
// TMA tile load without hardware swizzle, through a four-dimensional view of the pool (64 values,
// 8 rows, the halves of a row, groups of 8 rows): it lands as [group of 8 keys][half][8 rows][128
// bytes], which the tensor cores read directly with a stride of NHALF * 1024 bytes from one group
// of 8 rows to the next: K-major for Q K^T (the other half of the head 1024 bytes further), MN-major
// (rows are the k of the product) for P V (the other 64 columns of the head 1024 bytes further).
// Q comes from the step's plain [tokens, heads, head_dim] buffer through a three-dimensional map with
// the hardware swizzle.
//
// Every wait is bounded (status bit 128 when one ran out).
#include "tcgen05.cuh"

using namespace tc;

struct AttnWork { int seg, q_token0, q_count, q_pos0, kv_begin, kv_end, part_slot, split; };

namespace {

// Key tiles (and as many value tiles) in flight: an even number, two tiles are used at a time.
#ifndef PLLM_ATT_STAGES
#define PLLM_ATT_STAGES 4
#endif
// Softmax groups that take the key tiles in turn: four warps each.
#define PLLM_ATT_GROUPS 2
// After how many of a tile's 32 pairs of weights a group lets the other begin with its exponentials
#ifndef PLLM_ATT_HANDOVER
#define PLLM_ATT_HANDOVER 32
#endif
constexpr int P_G = PLLM_ATT_GROUPS;
constexpr int P_ROWS = 128, P_BK = 64, P_STAGES = PLLM_ATT_STAGES, P_THREADS = (4 * P_G + 8) * 32;
constexpr int W_KEYS = 4 * P_G, W_SCORES = 4 * P_G + 1, W_VALUES = 4 * P_G + 2, W_SUMS = 4 * P_G + 3;
constexpr int W_KEYS2 = 4 * P_G + 4, W_VALUES2 = 4 * P_G + 5;    // the producers of the odd tiles
constexpr int W_SCORES2 = 4 * P_G + 6, W_SUMS2 = 4 * P_G + 7;   // the second group's issuing threads
static_assert(P_G == 2 && P_STAGES % 2 == 0, "the register split and the producers' turns are laid out for two groups and an even ring");   // the other four warps   // P_STAGES: key tiles, and as many value tiles, in flight
constexpr float P_RESCALE = 8.0f;              // log2 units the running maximum may lag behind

__device__ __forceinline__ float max3(float a, float b, float c) {
    float y;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
    return y;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace

// A build for finding who waits for whom (-DPLLM_ATT_CLOCKS=1): one thread of each role adds up the
// clocks it spends in each of its waits and in its own work, and leaves the sums in a buffer that
// pllm_attention_prefill_clocks_read copies out: [work item < 64][role][slot], for kv head 0.
#ifdef PLLM_ATT_CLOCKS
static __device__ long long g_att_clocks[64][10][8];
static __device__ long long g_att_events[8][128][4];      // [role][tile][event] clock of work item 0, kv head 0
#define EVT(role, tile, slot) { if (blockIdx.y == 0 && blockIdx.x == 0 && (tile) < 128) g_att_events[role][tile][slot] = clock64(); }
PLLM_EXPORT int pllm_attention_prefill_events_read(long long* out) {
    cudaDeviceSynchronize();
    return (int)cudaMemcpyFromSymbol(out, g_att_events, sizeof(g_att_events));
}
#define CLK_BEGIN long long clk_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long clk_t = clock64();
#define CLK(slot) { const long long clk_n = clock64(); clk_acc[slot] += clk_n - clk_t; clk_t = clk_n; }
#define CLK_END(role) if (blockIdx.y < 64 && blockIdx.x == 0) { for (int ci = 0; ci < 8; ci++) g_att_clocks[blockIdx.y][role][ci] = clk_acc[ci]; }
PLLM_EXPORT int pllm_attention_prefill_clocks_read(long long* out) {
    cudaDeviceSynchronize();
    return (int)cudaMemcpyFromSymbol(out, g_att_clocks, sizeof(g_att_clocks));
}
#else
#define CLK_BEGIN
#define CLK(slot)
#define CLK_END(role)
#define EVT(role, tile, slot) {}
#endif

template <int HD>
__global__ void __launch_bounds__(P_THREADS, 1) attention_prefill_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, const int* __restrict__ block_tables, const AttnWork* __restrict__ work,
    const int* __restrict__ n_work_ptr, bf16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    int nh, int nkv, int page_size, int page_shift, int n_pages, int table_width, float scale_log2, int heads_per_cta,
    int tile_tokens, int take_single, int* status) {
    constexpr int NHALF = HD / 64;
    constexpr int GROUP = NHALF * 1024;            // 8 keys (or values): [half][8 rows][128 bytes]
    constexpr int Q_BYTES = NHALF * P_ROWS * 128, STAGE = (P_BK / 8) * GROUP;   // STAGE: a key (or value) tile
    // Tensor memory: two buffers of scores a group (64 columns each; the tile's weights, two to a column, are
    // written over the first 32 of the scores they came from), then head_dim columns of O a group.
    constexpr uint32_t S_COL = 0, O_COL = 2 * P_G * P_BK;
    constexpr uint32_t TMEM_USED = O_COL + P_G * HD, TMEM_COLS = TMEM_USED <= 256 ? 256 : 512;
    static_assert(TMEM_USED <= 512, "tensor memory has 512 columns");
    if ((int)blockIdx.y >= *n_work_ptr) return;
    const AttnWork w = work[blockIdx.y];
    // single decoded tokens are another kernel's, unless this one is told to take them too (a step of
    // portions beside a few decoded tokens: one launch instead of two; their rows are few, their keys the same)
    if (w.q_count <= 1 && !take_single) return;
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
    const uint32_t k_ring = q_s + Q_BYTES, v_ring = k_ring + P_STAGES * STAGE;
    constexpr int RINGS = 2 * P_STAGES * STAGE;
    // [groups][128] the groups' maxima and sums at the end, in the queries' place: written only when every
    // product has run (o_full)
    float* mstate = reinterpret_cast<float*>(smem);
    float* lpart = mstate + P_G * P_ROWS;
    static_assert(2 * P_G * P_ROWS * 4 <= Q_BYTES, "the groups' maxima and sums lie in the queries' place");
    unsigned char* ctl = smem + Q_BYTES + RINGS;
    const uint32_t bars = smem_u32(ctl);
    const uint32_t q_full = bars, k_full = bars + 8, k_empty = k_full + 8 * P_STAGES, v_full = k_empty + 8 * P_STAGES,
                   v_empty = v_full + 8 * P_STAGES, s_full = v_empty + 8 * P_STAGES,      // s_full, p_full, p_empty: [group][buffer]
                   p_full = s_full + 16 * P_G, p_empty = p_full + 16 * P_G, o_full = p_empty + 16 * P_G,
                   turn = o_full + 8;
    constexpr int N_BARS = 4 * P_STAGES + 1 + 6 * P_G + 1 + P_G;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctl + 8 * N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ctl + 8 * N_BARS + 8);

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < P_STAGES; s++) {
            mbar_init(k_full + 8 * s, 1); mbar_init(k_empty + 8 * s, 1);
            mbar_init(v_full + 8 * s, 1); mbar_init(v_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2 * P_G; b++) {
            mbar_init(s_full + 8 * b, 1);
            mbar_init(p_full + 8 * b, 4);        // one arrival from each warp of the group
            mbar_init(p_empty + 8 * b, 1);
        }
        for (int b = 0; b < P_G; b++) mbar_init(turn + 8 * b, 4);          // the other group is through with its exponentials
        mbar_init(o_full, P_G);                  // each group's issuing thread, after its last product
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
        fence_async_smem();
    }
    if (warp == W_SCORES) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // Registers follow the work: the softmax threads hold a row of scores and weights each, the other
    // eight warps a few addresses (512 threads start with 128 registers each).
    // (The two halves of the CTA below each begin with their setmaxnreg: the compiler then knows the budget of
    // the code behind it, and the four warps of a group execute one and the same instruction.)
    if (warp >= 4 * P_G) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;\n" ::);
    if (warp == W_KEYS || warp == W_VALUES || warp == W_KEYS2 || warp == W_VALUES2) {
        // ---- producers: warp 8 the queries and the key tiles, warp 10 the value tiles, each with a ring
        // of its own (a key tile's place comes free when its scores are formed, two tiles before its
        // values' does; with one ring for both the keys would be fetched only two tiles ahead) --------
        // (a request costs the issuing warp 135 clocks, 540 a tile of four pages: two warps a ring, taking the tiles in turn)
        const bool keys = warp == W_KEYS || warp == W_KEYS2;
        const int first = (warp == W_KEYS || warp == W_VALUES) ? 0 : 1;
        const CUtensorMap* map = keys ? &map_k : &map_v;
        const uint32_t ring = keys ? k_ring : v_ring, full = keys ? k_full : v_full, empty = keys ? k_empty : v_empty;
        unsigned char* ring_ptr = smem + Q_BYTES + (keys ? 0 : P_STAGES * STAGE);
        const int slab_rows = page_size < P_BK ? page_size : P_BK;
        const int slabs = P_BK / slab_rows;                  // at most 8
        const uint32_t slab_bytes = (uint32_t)(slab_rows / 8) * GROUP;   // a page's rows of this tile, both halves
        const int* table = block_tables + (size_t)w.seg * table_width;
        // the table entries of the key range, 32 at a time, one in each lane, fetched ahead
        int win0 = w.kv_begin >> page_shift;
        int tbl = (win0 + lane < table_width) ? table[win0 + lane] : -1;
        // (the block table is the host's: fetched before the wait)
        pdl_wait(KID_ATT_TC, warp == W_KEYS && lane == 0);           // the queries and this step's cache rows come from the kernel before
        if (warp == W_KEYS && lane == 0) {
            mbar_expect_tx(q_full, (uint32_t)(NHALF * 128 * heads_per_cta * tile_tokens));
            for (int h = 0; h < NHALF; h++) tma_load_3d(q_s + h * P_ROWS * 128, &map_q, h * 64, head0, w.q_token0, q_full);
        }
        CLK_BEGIN
        for (int t = first; t < n_tiles; t += 2) {
            const int s = t % P_STAGES;
            const int kv0 = w.kv_begin + t * P_BK;
            if (((kv0 + P_BK - 1) >> page_shift) >= win0 + 32) {
                win0 = kv0 >> page_shift;
                tbl = (win0 + lane < table_width) ? table[win0 + lane] : -1;
            }
            // lane i takes slab i: its page out of the window
            const int jl = kv0 + (lane < slabs ? lane : 0) * slab_rows;
            int page = __shfl_sync(0xffffffffu, tbl, ((jl >> page_shift) - win0) & 31);
            if (lane >= slabs || jl >= w.kv_end) page = -1;
            if (page >= n_pages) { atomicOr(status, 8); page = -1; }
            CLK(1)
            if (t >= P_STAGES && !mbar_wait(empty + 8 * s, ((t / P_STAGES) - 1) & 1, abort_flag)) break;
            CLK(0)
            if (lane == 0) EVT(keys ? 4 : 5, t, 0)
            const uint32_t have = __ballot_sync(0xffffffffu, page >= 0) & ((1u << slabs) - 1);
            const uint32_t st_base = ring + s * STAGE;
            unsigned char* st_ptr = ring_ptr + s * STAGE;
            if (have != (1u << slabs) - 1) {
                // slabs with no page behind them are zeroed by hand: nothing stale is multiplied
                for (int i = 0; i < slabs; i++) {
                    if (have & (1u << i)) continue;
                    for (int o = lane * 16; o < (int)slab_bytes; o += 32 * 16)
                        *reinterpret_cast<uint4*>(st_ptr + i * slab_bytes + o) = make_uint4(0, 0, 0, 0);
                }
                fence_async_smem();
                __syncwarp();
            }
            if (lane == 0) mbar_expect_tx(full + 8 * s, slab_bytes * __popc(have));
            __syncwarp();
            CLK(2)
            // (One request a lane in one instruction: the same requests one after the other from an elected lane took
            //  the warp 277 clocks each, against 135 this way.)
            if (lane < slabs && page >= 0) {
                const int row = (page * nkv + kh) * page_size + (jl & (page_size - 1));
                tma_load_4d(st_base + lane * slab_bytes, map, 0, 0, 0, row >> 3, full + 8 * s);     // (a page starts on a multiple of 8 rows)
            }
            if (lane == 0) EVT(keys ? 4 : 5, t, 1)
        }
        if (lane == 0) { CLK(1) CLK_END((keys ? 4 : 5) + 2 * first) }
    } else if (warp == W_SCORES || warp == W_SCORES2) {
        // ---- tensor-core issue, the scores of one group's tiles: S[g] = Q K_t^T for t = g, g + 2, ...  Each
        // group has issuing threads of its own (this one and one for O += P V), so that nothing ties one
        // group's turn to the other's: they drift apart until one computes its exponentials while the
        // other loads, stores and waits.
        if (lane == 0) {
            const int g = warp == W_SCORES ? 0 : 1;
            constexpr uint32_t idesc_qk = instr_desc(P_ROWS, P_BK);
            // descriptors differ only in their address field (bits 0-13, units of 16 bytes): the rest is
            // made once, and an address offset is one addition
            const uint64_t q_desc = smem_desc(q_s), k_desc = smem_desc(k_ring, 16, GROUP);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            CLK_BEGIN
            for (int t = g; t < n_tiles && ok; t += P_G) {
                const int s = t % P_STAGES;
                const int k = t / P_G, buf = g * 2 + (k & 1);        // the group's k-th tile, into the buffer of its parity
                // (the key tile first: it is there long before, and a wait on a barrier that is over still
                // costs this thread a hundred clocks or two)
                if (!mbar_wait(k_full + 8 * s, (t / P_STAGES) & 1, abort_flag)) { ok = false; break; }
                CLK(1)
                EVT(0, t, 1)
                // the buffer held the scores and then the weights of the group's tile before last: those weights
                // must have gone into O.  (The scores are thus formed a whole turn of the group ahead.)
                if (k >= 2 && !mbar_wait(p_empty + 8 * buf, ((k >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
                CLK(0)
                EVT(0, t, 0)
                tc_fence_after();
                const uint64_t kd = k_desc + (uint64_t)((s * STAGE) >> 4);
                const uint32_t d = tmem + S_COL + buf * P_BK;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++)
                    mma_ss(d, q_desc + (uint64_t)(((ks / 4) * P_ROWS * 128 + (ks % 4) * 32) >> 4),
                           kd + (uint64_t)(((ks / 4) * 1024 + (ks % 4) * 32) >> 4), idesc_qk, ks ? 1u : 0u);
                mma_commit(s_full + 8 * buf);
                mma_commit(k_empty + 8 * s);         // the key tile's place is free once these have read it
                CLK(2)
                EVT(0, t, 2)
            }
            CLK_END(g ? 8 : 0)
        }
    } else if (warp == W_SUMS || warp == W_SUMS2) {
        // ---- tensor-core issue, the sums of one group's tiles: O[g] += P_t V_t --------------------------
        if (lane == 0) {
            const int g = warp == W_SUMS ? 0 : 1;
            constexpr uint32_t idesc_pv = instr_desc(P_ROWS, HD, 1);
            const uint64_t v_desc = smem_desc(v_ring, 1024, GROUP);
            bool ok = true;
            CLK_BEGIN
            for (int t = g; t < n_tiles && ok; t += P_G) {
                const int k = t / P_G, buf = g * 2 + (k & 1);
                if (!mbar_wait(v_full + 8 * (t % P_STAGES), (t / P_STAGES) & 1, abort_flag)) { ok = false; break; }      // (the values first, likewise)
                CLK(1)
                EVT(1, t, 1)
                if (!mbar_wait(p_full + 8 * buf, (k >> 1) & 1, abort_flag)) { ok = false; break; }
                CLK(0)
                EVT(1, t, 0)
                tc_fence_after();
                const uint64_t vd = v_desc + (uint64_t)(((t % P_STAGES) * STAGE) >> 4);
#pragma unroll
                for (int ks = 0; ks < P_BK / 16; ks++)    // 16 keys = two groups of 8 rows
                    mma_ts(tmem + O_COL + g * HD, tmem + S_COL + buf * P_BK + ks * 8, vd + (uint64_t)((ks * 2 * GROUP) >> 4), idesc_pv,
                           (k || ks) ? 1u : 0u);
                mma_commit(p_empty + 8 * buf);               // the weights are read: O holds the tile, the buffer may take new scores
                mma_commit(v_empty + 8 * (t % P_STAGES));    // and so are the values of this tile
                CLK(2)
                EVT(1, t, 2)
            }
            CLK_END(g ? 9 : 1)
            if (ok) mma_commit(o_full);                      // (one arrival from each group's thread)
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 192;\n" ::);
        // ---- softmax, one row a thread, the two groups taking the tiles in turn; then the epilogue ----
        pdl_launch_dependents();
        const int grp = warp >> 2, wq = warp & 3;
        const int row = wq * 32 + lane;
        const int tq = row / heads_per_cta, hh = row % heads_per_cta;
        const bool live = tq < w.q_count && hh < n_heads && tq < tile_tokens;
        // keys below hi are visible to this row; rows that are no query's see everything (their
        // results are never stored, and a row of nothing but masked keys would make NaN)
        const int hi = live ? min(w.kv_end, w.q_pos0 + tq + 1) : w.kv_end;
        const uint32_t lane_base = tmem + ((uint32_t)(wq * 32) << 16);
        // this group's part of the row's sum, in units of 2^m_ref
        float m_ref = -CUDART_INF_F, l_run = 0.f;
        bool ok = true;
        // The exponentials of the two groups take turns (they share one unit, and left alone the groups fall
        // into step: both compute theirs at once, at half speed each, and then both wait): a group computes
        // its tile's when the other is through with those of the tile before, and meanwhile loads, stores and waits.
        if (grp == 1 && lane == 0) mbar_arrive(turn);
        CLK_BEGIN
        for (int t = grp; t < n_tiles; t += P_G) {
            const int kv0 = w.kv_begin + t * P_BK;
            const int k = t / P_G, buf = grp * 2 + (k & 1);      // the group's k-th tile, in the buffer of its parity
            if (!mbar_wait(s_full + 8 * buf, (k >> 1) & 1, abort_flag)) { ok = false; break; }
            CLK(0)
            if (wq == 0 && lane == 0) EVT(2 + grp, t, 0)
            tc_fence_after();
            uint32_t v0[32], v1[32];
            tmem_ld32(lane_base + S_COL + buf * P_BK, v0);
            tmem_ld32(lane_base + S_COL + buf * P_BK + 32, v1);
            tmem_wait_ld();
            CLK(1)
            // keys of this tile at or past vis are hidden from this row (only tiles on the diagonal have any)
            const int vis = hi - kv0;
            if (vis < P_BK) {
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    if (i >= vis) v0[i] = 0xff800000u;          // -inf
                    if (i + 32 >= vis) v1[i] = 0xff800000u;
                }
            }
            // the row's maximum, four chains side by side, three numbers to an instruction
            float m4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
#pragma unroll
                for (int c = 0; c < 4; c++) m4[c] = max3(m4[c], __uint_as_float(v0[i + c]), __uint_as_float(v1[i + c]));
            }
            const float mx = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])) * scale_log2;   // the scale is positive
            // the maximum this group has in use; it moves only when it grew by more than 2^8 (or is not set yet)
            const float m_prev = m_ref;
            CLK(2)
            const bool grow = mx > m_prev + P_RESCALE || (m_prev == -CUDART_INF_F && mx > -CUDART_INF_F);
            const float m_used = grow ? mx : m_prev;
            CLK(3)
            if (wq == 0 && lane == 0) EVT(2 + grp, t, 1)
            if (k >= 1 && __any_sync(0xffffffffu, grow)) {
                // this group's O is rescaled once its tile before this one is in it (this tile's is not issued
                // before the group has stored its weights)
                if (!mbar_wait(p_empty + 8 * (buf ^ 1), ((k - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const float alpha = (grow && m_prev > -CUDART_INF_F) ? ex2(m_prev - m_used) : (grow ? 0.f : 1.f);
#pragma unroll
                for (int c = 0; c < HD / 32; c++) {
                    uint32_t o[32];
                    tmem_ld32(lane_base + O_COL + grp * HD + c * 32, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_base + O_COL + grp * HD + c * 32, o);
                }
                tmem_wait_st();
            }
            CLK(4)
            // this group's sum so far, brought to the maximum now in use
            if (m_ref != m_used) {
                l_run = m_ref > -CUDART_INF_F ? l_run * ex2(m_ref - m_used) : 0.f;
                m_ref = m_used;
            }
            if (!mbar_wait(turn + 8 * grp, (t / P_G) & 1, abort_flag)) { ok = false; break; }
            // weights 2^(s * scale - m): one multiply-add and one exponential each; a hidden key's -inf gives 0
            const float neg_m = m_used > -CUDART_INF_F ? -m_used : 0.f;
            uint32_t pw[32];
            // (eight sums side by side, each weight added to one of them directly: with four, and a pair's sum
            //  formed first, a warp alone on its scheduler took 1083 clocks for these 64 weights instead of 704,
            //  which is what the 64 exponentials take by themselves)
            float s8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 32; i++) {
                const uint32_t a = i < 16 ? v0[2 * i] : v1[2 * i - 32], b2 = i < 16 ? v0[2 * i + 1] : v1[2 * i - 31];
                const float p0 = ex2(fmaf(__uint_as_float(a), scale_log2, neg_m));
                const float p1 = ex2(fmaf(__uint_as_float(b2), scale_log2, neg_m));
                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                pw[i] = *reinterpret_cast<uint32_t*>(&h);
                s8[2 * (i & 3)] += p0;
                s8[2 * (i & 3) + 1] += p1;
                if (i == PLLM_ATT_HANDOVER - 1) {
                    // the other group may begin: it takes a hundred clocks or two to notice
                    __syncwarp();
                    if (lane == 0 && t + 1 < n_tiles) mbar_arrive(turn + 8 * (grp ^ 1));
                }
            }
            l_run += ((s8[0] + s8[1]) + (s8[2] + s8[3])) + ((s8[4] + s8[5]) + (s8[6] + s8[7]));
            CLK(5)
            if (wq == 0 && lane == 0) EVT(2 + grp, t, 2)
            CLK(6)
            // the row's 64 weights, two to a column, over the first 32 of the scores they came from (this thread's
            // lane: nobody else's scores)
            tmem_st32(lane_base + S_COL + buf * P_BK, pw);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * buf);
            CLK(7)
            if (wq == 0 && lane == 0) EVT(2 + grp, t, 3)
        }
        if (wq == 0 && lane == 0) { CLK_END(2 + grp) }
        // ---- the groups meet: each has a maximum, a sum and an O of its own (the even tiles', the odd tiles'),
        // brought to the larger maximum here; each group stores half of the columns ------------------------
        if (!ok || *abort_flag) *abort_flag = 1;
        const bool have_o = !*abort_flag && mbar_wait(o_full, 0, abort_flag);      // (the last product has read Q, the keys and the values)
        mstate[grp * P_ROWS + row] = m_ref;
        lpart[grp * P_ROWS + row] = l_run;
        asm volatile("bar.sync 1, %0;\n" ::"n"(P_G * 128) : "memory");          // (the softmax warps; the others are elsewhere)
        float m_fin = mstate[row];
#pragma unroll
        for (int g = 1; g < P_G; g++) m_fin = fmaxf(m_fin, mstate[g * P_ROWS + row]);
        float share[P_G], l_tot = 0.f;        // 2^(a group's maximum - the row's): 0 for a group that saw no key of this row
#pragma unroll
        for (int g = 0; g < P_G; g++) {
            const float mg = mstate[g * P_ROWS + row], lg = lpart[g * P_ROWS + row];
            share[g] = (g < n_tiles && mg > -CUDART_INF_F && lg > 0.f) ? ex2(mg - m_fin) : 0.f;
            l_tot += share[g] > 0.f ? lg * share[g] : 0.f;
        }
        if (have_o && !*abort_flag) {
            tc_fence_after();
            const float inv = l_tot > 0.f ? 1.0f / l_tot : 0.f;
            // chunks of 32 columns, dealt to the groups
            for (int c = grp; c < HD / 32; c += P_G) {
                uint32_t o[32];
                tmem_ld32(lane_base + O_COL + c * 32, o);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; i++) o[i] = __float_as_uint(share[0] > 0.f ? __uint_as_float(o[i]) * share[0] : 0.f);
#pragma unroll
                for (int g = 1; g < P_G; g++) {
                    if (g >= n_tiles) continue;          // (a group without a tile never wrote its O)
                    uint32_t og[32];
                    tmem_ld32(lane_base + O_COL + g * HD + c * 32, og);
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (share[g] > 0.f) o[i] = __float_as_uint(__uint_as_float(o[i]) + __uint_as_float(og[i]) * share[g]);
                }
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
                    if (c == 0) { part_ml[pr * 2] = m_fin * 0.6931471805599453f; part_ml[pr * 2 + 1] = l_tot; }   // natural-log units
                }
            }
        }
    }
    // ---- everyone meets; the allocating warp gives the tensor memory back ---------------------------
    tc_fence_before();
    __syncthreads();
    if (warp == W_SCORES) {
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
                          int nh, int nkv, int page_size, int n_pages, int table_width, float scale, int take_single,
                          int* status, cudaStream_t stream) {
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
        // the pool as (64 values, 8 rows, the halves of a row, groups of 8 rows): a box lands as [group][half][8 rows][128 bytes]
        const long long dp[4] = {64, 8, HD / 64, (long long)n_pages * nkv * page_size / 8}, sp[3] = {2LL * HD, 128, 16LL * HD};
        const int bp[4] = {64, 8, HD / 64, slab_rows / 8};
        if (tensor_map(k_pool, 4, dp, sp, bp, false, &map_k) != 0) return PLLM_ERR_SIZE;
        if (tensor_map(v_pool, 4, dp, sp, bp, false, &map_v) != 0) return PLLM_ERR_SIZE;
    }
    constexpr int NHALF = HD / 64;
    const size_t smem = (size_t)NHALF * P_ROWS * 128 + (size_t)P_STAGES * 2 * NHALF * P_BK * 128 +
                        8 * (4 * P_STAGES + 2 + 7 * P_G) + 16 + 1024;
    cudaFuncSetAttribute(attention_prefill_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(attention_prefill_tcgen05_kernel<HD>, dim3(nkv * gparts, max_work), dim3(P_THREADS), smem, stream, map_q,
                   map_k, map_v, block_tables, (const AttnWork*)work, n_work_ptr, (bf16*)out, part_o, part_ml, nh, nkv,
                   page_size, page_shift, n_pages, table_width, scale * 1.4426950408889634f, heads_per_cta, tile_tokens, take_single,
                   status);
    return launch_status();
}

// q, out: [n_tokens, nh, hd] bfloat16; pools [n_pages, nkv, page_size, hd] with swizzled rows.
PLLM_EXPORT int pllm_attention_prefill_tcgen05(const void* q, const void* k_pool, const void* v_pool, const int* block_tables,
                                               const int* work, const int* n_work_ptr, int max_work, void* out,
                                               float* part_o, float* part_ml, int n_tokens, int nh, int nkv, int hd,
                                               int page_size, int n_pages, int table_width, float scale, int take_single,
                                               int* status, cudaStream_t stream) {
    if (max_work <= 0 || n_tokens <= 0) return PLLM_OK;
    if (!pllm_attention_prefill_tcgen05_supports(PLLM_BF16, nh, nkv, hd, page_size, 0)) return PLLM_ERR_SIZE;
    if (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15) return PLLM_ERR_ALIGN;
    if (hd == 128)
        return launch_prefill<128>(q, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, n_tokens,
                                   nh, nkv, page_size, n_pages, table_width, scale, take_single, status, stream);
    return launch_prefill<64>(q, k_pool, v_pool, block_tables, work, n_work_ptr, max_work, out, part_o, part_ml, n_tokens, nh,
                              nkv, page_size, n_pages, table_width, scale, take_single, status, stream);
}

PLLM_TRACE_EXPORT(attention_prefill_tcgen05)

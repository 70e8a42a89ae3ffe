// y[M, N] = x[M, K] . W[N, K]^T in bfloat16 with float accumulation on the fifth-generation
// tensor cores, for the many rows of a prompt portion: tcgen05.mma issued by one thread,
// operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle), the
// accumulator in tensor memory, read back with tcgen05.ld for the epilogue.
//
// The reference calls a library product for every projection
// (crates/pagedllm/src/model/layers.rs:27-35) and a pass of its own for the gated
// activation (crates/pagedllm/src/model/layers.rs:93-99).  This kernel is the product with
// that activation in its epilogue: with GLU the weight is [gate rows | up rows] and a CTA
// multiplies 64 rows of each, so that y = silu(gate) * up leaves the kernel and the
// [M, 2N] intermediate is never written.
//
// A third form is the attention's input projection with what follows it in its epilogue
// (crates/pagedllm/src/model/attention.rs:148-158 in the reference: q and k normed per head,
// rotated at the token's position, k and v scattered into the cache, each a pass over the
// tensor): a tile's columns are whole heads and an epilogue thread holds one token's row of
// them, so the norm over a head and the rotation's pairs (d, d + head_dim / 2) need no other
// thread; q leaves as [tokens, heads * head_dim], k and v go straight to their cache rows,
// and the [tokens, (heads + 2 kv heads) * head_dim] intermediate is never written.
//
// The kernel is persistent: one CTA to an SM, each taking tiles of 128 x BN (BN = 256, or 128
// where the width asks for it) in turn, m fastest, so that the CTAs at work share W tiles in
// L2.  Six warps:
//   warp 4     producer: waits for a free stage, arms its barrier with the bytes to come and
//              issues the TMA loads (a 128 x 64 tile of x, a BN x 64 tile of W; GLU: BN/2 rows
//              of gate and of up)
//   warp 5     allocates tensor memory (two accumulators of BN columns); one lane waits for
//              a full stage and issues four tcgen05.mma (K = 16 each), then tcgen05.commit,
//              which frees the stage when those have read it; after a tile's last, a commit
//              to that accumulator's barrier
//   warps 0-3  epilogue: wait for an accumulator, tcgen05.ld their 32 lanes (= rows) 32
//              columns at a time, convert, (activation,) store, hand the accumulator back;
//              the tensor cores are on the next tile meanwhile
// Every wait is bounded: a thread that gives up raises a flag that the others see, the
// CTA frees its tensor memory and leaves, and the status word says so (bit 64).
#include "tcgen05.cuh"

using namespace tc;

namespace {

constexpr int G_BM = 128, G_BK = 64;
constexpr int G_TILE_A = G_BM * G_BK * 2;           // 16 KB
constexpr int G_SMEM_TILES = 192 * 1024;            // what the stages may fill
constexpr int G_THREADS = 192;
constexpr int G_EPI_BUF = 32 * 144 * 2;             // an epilogue warp's staging buffer (EPI == 2): 32 rows of 144 bytes, twice

}  // namespace

// What the epilogue of the attention's input projection needs (EPI == 2).
struct QkvEpilogue {
    bf16* q_out;                     // [M, nh * hd]
    bf16 *k_pool, *v_pool;           // [pages, nkv, page_size, hd], or null: keys and values are not kept
    const int* positions;            // [M]
    const int* slots;                // [M] page * page_size + offset, -1: no cache row for this token
    const float *q_gain, *k_gain;    // [hd] or null: no norm
    const float *cos_t, *sin_t;      // [max_pos, hd / 2] or null: no rotation
    float eps;
    int nh, nkv, page_size, n_pages, max_pos, swizzle;
};

// map_a: x [M, K], box 64 x 128.  map_b: W [rows, K], box 64 x BN (plain) or 64 x BN/2 (GLU).
// y: [M, n_out] bfloat16; n_out = N (plain) or N / 2 (GLU, W = [gate; up] of n_out rows each).
template <int EPI, int BN, int HD>
__global__ void __launch_bounds__(G_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                    const __grid_constant__ CUtensorMap map_b,
                                                                    bf16* __restrict__ y, int M, int n_out, int K,
                                                                    const QkvEpilogue e, int* status) {
    constexpr bool GLU = EPI == 1;
    constexpr int TILE_B = BN * G_BK * 2, STAGE = G_TILE_A + TILE_B;
    constexpr int STAGES = (G_SMEM_TILES - (EPI == 2 ? 4 * G_EPI_BUF : 0)) / STAGE;
    constexpr int OUT_BN = GLU ? BN / 2 : BN;            // columns of y a tile makes
    constexpr uint32_t TMEM_COLS = 2 * BN;               // two accumulators
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the tiles need 1024-byte alignment for the 128-byte swizzle
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const uint32_t tiles = smem_u32(smem);
    unsigned char* ctl = smem + STAGES * STAGE;
    const uint32_t bars = smem_u32(ctl);                 // full[S], empty[S], acc_full[2], acc_empty[2]
    const uint32_t acc_full = bars + 8 * 2 * STAGES, acc_empty = acc_full + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctl + 8 * (2 * STAGES + 4));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ctl + 8 * (2 * STAGES + 4) + 8);
    unsigned char* epi_buf = ctl + 8 * (2 * STAGES + 4) + 16;     // [4 warps][G_EPI_BUF] (EPI == 2)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + G_BM - 1) / G_BM, tiles_n = n_out / OUT_BN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_blocks = (K + G_BK - 1) / G_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bars + 8 * s, 1);
            mbar_init(bars + 8 * (STAGES + s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full + 8 * b, 1);
            mbar_init(acc_empty + 8 * b, 4);     // one arrival from each epilogue warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::);
        asm volatile("fence.proxy.async.shared::cta;\n" ::);
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
        // ---- producer ---------------------------------------------------------------------------
        if (lane == 0) {
            pdl_wait(KID_GEMM_TC, true);      // x comes from the kernel before this one
            int it = 0;      // k blocks loaded so far, over all of this CTA's tiles
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x) {
                const int m0 = (t % tiles_m) * G_BM, n0 = (t / tiles_m) * OUT_BN;
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(bars + 8 * (STAGES + s), ((it / STAGES) - 1) & 1, abort_flag)) { ok = false; break; }
                    const uint32_t a_dst = tiles + s * STAGE, b_dst = a_dst + G_TILE_A;
                    mbar_expect_tx(bars + 8 * s, STAGE);
                    tma_load_2d(a_dst, &map_a, kb * G_BK, m0, bars + 8 * s);
                    if (GLU) {
                        tma_load_2d(b_dst, &map_b, kb * G_BK, n0, bars + 8 * s);                        // gate rows
                        tma_load_2d(b_dst + TILE_B / 2, &map_b, kb * G_BK, n_out + n0, bars + 8 * s);   // up rows
                    } else {
                        tma_load_2d(b_dst, &map_b, kb * G_BK, n0, bars + 8 * s);
                    }
                }
            }
        }
    } else if (warp == 5) {
        // ---- tensor-core issue ------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(G_BM, BN);
            int it = 0, i = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < n_tiles && ok; t += gridDim.x, i++) {
                const int b = i & 1;
                // the epilogue must have read this accumulator's last tile out
                if (i >= 2 && !mbar_wait(acc_empty + 8 * b, ((i >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                for (int kb = 0; kb < k_blocks; kb++, it++) {
                    const int s = it % STAGES;
                    if (!mbar_wait(bars + 8 * s, (it / STAGES) & 1, abort_flag)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_src = tiles + s * STAGE, b_src = a_src + G_TILE_A;
#pragma unroll
                    for (int j = 0; j < G_BK / 16; j++)   // 16 values of k = 32 bytes along the swizzled row
                        mma_ss(tmem + b * BN, smem_desc(a_src + j * 32), smem_desc(b_src + j * 32), idesc, (kb | j) ? 1u : 0u);
                    mma_commit(bars + 8 * (STAGES + s));      // the stage is free once these have read it
                }
                if (ok) mma_commit(acc_full + 8 * b);         // this tile's accumulator is complete
            }
        }
    } else {
        // ---- epilogue: warp w owns lanes (rows) 32 w .. 32 w + 31 of the accumulators ---------------
        pdl_launch_dependents();
        int i = 0;
        for (int t = blockIdx.x; t < n_tiles; t += gridDim.x, i++) {
            const int b = i & 1;
            const int m0 = (t % tiles_m) * G_BM, n0 = (t / tiles_m) * OUT_BN;
            if (!mbar_wait(acc_full + 8 * b, (i >> 1) & 1, abort_flag)) break;
            tc_fence_after();
            const int row = m0 + warp * 32 + lane;
            const uint32_t acc = tmem + ((uint32_t)(warp * 32) << 16) + b * BN;
            if constexpr (EPI == 2) {
                // ---- this thread's token, BN / HD heads of it: norm, rotation, q out, k and v to the cache ----
                constexpr int HEADS = BN / HD, HC = HD / 32, HALF = HC / 2;
                const bool live = row < M;
                int pos = 0, slot = -1;
                if (live) {
                    pos = e.positions[row];
                    if (e.slots) slot = e.slots[row];
                    if (e.cos_t && (pos < 0 || pos >= e.max_pos)) { atomicOr(status, 4); pos = 0; }
                }
#pragma unroll 1
                for (int hh = 0; hh < HEADS; hh++) {
                    const int head = n0 / HD + hh;                       // among nh + 2 nkv
                    const int kind = head < e.nh ? 0 : (head < e.nh + e.nkv ? 1 : 2);
                    const uint32_t hacc = acc + hh * HD;
                    const float* gain = kind == 0 ? e.q_gain : (kind == 1 ? e.k_gain : nullptr);
                    // the values rounded as the product alone would leave them, then the arithmetic of
                    // qk_norm_rope_kv.cu in float
                    float inv = 1.f;
                    if (gain) {
                        float ss = 0.f;
#pragma unroll 1
                        for (int c = 0; c < HC; c++) {
                            uint32_t v[32];
                            tmem_ld32(hacc + c * 32, v);
                            tmem_wait_ld();
#pragma unroll
                            for (int k = 0; k < 32; k++) { const float f = round_bf16(__uint_as_float(v[k])); ss = fmaf(f, f, ss); }
                        }
                        inv = 1.0f / sqrtf(ss / (float)HD + e.eps);
                    }
                    bf16* dst = nullptr;
                    int xr = 0;        // what a cache row's 16-byte chunks are XOR-ed with
                    if (live) {
                        if (kind == 0) {
                            dst = e.q_out + ((size_t)row * e.nh + head) * HD;
                        } else if (slot >= 0 && e.k_pool) {
                            const int page = slot / e.page_size, off = slot % e.page_size;
                            if (page >= e.n_pages) {
                                atomicOr(status, 2);
                            } else {
                                const int kh = kind == 1 ? head - e.nh : head - e.nh - e.nkv;
                                dst = (kind == 1 ? e.k_pool : e.v_pool) + (((size_t)page * e.nkv + kh) * e.page_size + off) * HD;
                                if (e.swizzle) xr = off & 7;
                            }
                        }
                    }
                    const bool rot = kind != 2 && e.cos_t != nullptr;
                    // A thread holds a token's row, so a load or store of a warp would touch 32 lines, 16 bytes of
                    // each.  Rotation factors and results go through a buffer of the warp's own in shared memory
                    // instead, so that global memory sees whole 64- and 128-byte runs.
                    unsigned char* buf = epi_buf + warp * G_EPI_BUF;
                    const uint32_t dst_lo = (uint32_t)(uintptr_t)dst, dst_hi = (uint32_t)((uintptr_t)dst >> 32);
#pragma unroll 1
                    for (int c = 0; c < HALF; c++) {
                        float co[32], si[32];
                        if (rot) {
                            // rows 4 j .. 4 j + 3 of the warp's 32, eight lanes (128 bytes) to each, by the row's own position
                            float* tab = reinterpret_cast<float*>(buf);          // [2][32][36]
#pragma unroll
                            for (int j = 0; j < 8; j++) {
                                const int r = 4 * j + (lane >> 3);
                                const int pr = __shfl_sync(0xffffffffu, pos, r);
                                const size_t at = (size_t)pr * (HD / 2) + c * 32 + (lane & 7) * 4;
                                *reinterpret_cast<float4*>(tab + r * 36 + (lane & 7) * 4) = __ldg(reinterpret_cast<const float4*>(e.cos_t + at));
                                *reinterpret_cast<float4*>(tab + (32 + r) * 36 + (lane & 7) * 4) = __ldg(reinterpret_cast<const float4*>(e.sin_t + at));
                            }
                            __syncwarp();
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const float4 cv = *reinterpret_cast<const float4*>(tab + lane * 36 + i * 4);
                                const float4 sv = *reinterpret_cast<const float4*>(tab + (32 + lane) * 36 + i * 4);
                                co[4 * i] = cv.x; co[4 * i + 1] = cv.y; co[4 * i + 2] = cv.z; co[4 * i + 3] = cv.w;
                                si[4 * i] = sv.x; si[4 * i + 1] = sv.y; si[4 * i + 2] = sv.z; si[4 * i + 3] = sv.w;
                            }
                            __syncwarp();
                        }
                        uint32_t lo[32], hi[32];
                        tmem_ld32(hacc + c * 32, lo);
                        tmem_ld32(hacc + (c + HALF) * 32, hi);
                        tmem_wait_ld();
                        if (hh == HEADS - 1 && c == HALF - 1) {
                            // the accumulator's last values are in registers: the tensor cores may have it back
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(acc_empty + 8 * b);
                        }
                        // this row's 64 bytes of the lower half and of the upper half of the head, the 16-byte chunks
                        // already where the cache's swizzle wants them inside their run of four
                        uint4* st = reinterpret_cast<uint4*>(buf);                // [32][9]: lo 0-3, hi 4-7
#pragma unroll
                        for (int k8 = 0; k8 < 32; k8 += 8) {
                            const int d0 = c * 32 + k8;
                            float a[8], bb[8];
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                a[i] = round_bf16(__uint_as_float(lo[k8 + i]));
                                bb[i] = round_bf16(__uint_as_float(hi[k8 + i]));
                            }
                            if (gain) {
                                const float4 g0 = __ldg(reinterpret_cast<const float4*>(gain + d0)), g1 = __ldg(reinterpret_cast<const float4*>(gain + d0 + 4));
                                const float4 h0 = __ldg(reinterpret_cast<const float4*>(gain + d0 + HD / 2)), h1 = __ldg(reinterpret_cast<const float4*>(gain + d0 + HD / 2 + 4));
                                const float ga[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                                const float gb[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
                                for (int i = 0; i < 8; i++) { a[i] = a[i] * inv * ga[i]; bb[i] = bb[i] * inv * gb[i]; }
                            }
                            if (rot) {
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    const float x1 = a[i], x2 = bb[i];
                                    a[i] = x1 * co[k8 + i] - x2 * si[k8 + i];
                                    bb[i] = x2 * co[k8 + i] + x1 * si[k8 + i];
                                }
                            }
                            const int q4 = (k8 >> 3) ^ (xr & 3);
                            st[lane * 9 + q4] = make_uint4(pack2(a[0], a[1]), pack2(a[2], a[3]), pack2(a[4], a[5]), pack2(a[6], a[7]));
                            st[lane * 9 + 4 + q4] = make_uint4(pack2(bb[0], bb[1]), pack2(bb[2], bb[3]), pack2(bb[4], bb[5]), pack2(bb[6], bb[7]));
                        }
                        __syncwarp();
                        // out: rows 4 j .. 4 j + 3, four lanes to each run of 64 bytes
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            const int r = 4 * j + (lane >> 3), seg = (lane >> 2) & 1, q4 = lane & 3;
                            const uint4 v = st[r * 9 + seg * 4 + q4];
                            const uint32_t plo = __shfl_sync(0xffffffffu, dst_lo, r), phi = __shfl_sync(0xffffffffu, dst_hi, r);
                            const int xrr = __shfl_sync(0xffffffffu, xr, r);
                            bf16* drow = reinterpret_cast<bf16*>(((uintptr_t)phi << 32) | plo);
                            const int first = ((seg ? c + HALF : c) * 4) ^ (xrr & 4);      // the run's first chunk in the row
                            if (drow) *reinterpret_cast<uint4*>(drow + ((first + q4) << 3)) = v;
                        }
                        __syncwarp();
                    }
                }
            } else {
#pragma unroll 2
            for (int c = 0; c < OUT_BN / 32; c++) {
                uint32_t v[32], out[16];
                tmem_ld32(acc + c * 32, v);
                if (GLU) {
                    uint32_t u[32];
                    tmem_ld32(acc + BN / 2 + c * 32, u);
                    tmem_wait_ld();
#pragma unroll
                    for (int k = 0; k < 16; k++) {
                        // gate and up rounded as a product of their own would leave them, then the activation
                        const float g0 = round_bf16(__uint_as_float(v[2 * k])), g1 = round_bf16(__uint_as_float(v[2 * k + 1]));
                        const float u0 = round_bf16(__uint_as_float(u[2 * k])), u1 = round_bf16(__uint_as_float(u[2 * k + 1]));
                        // (fast exponential and division: their error is far below the rounding to bfloat16,
                        //  and the epilogue must keep pace with the tensor cores)
                        out[k] = pack2(__fdividef(g0, 1.0f + __expf(-g0)) * u0, __fdividef(g1, 1.0f + __expf(-g1)) * u1);
                    }
                } else {
                    tmem_wait_ld();
#pragma unroll
                    for (int k = 0; k < 16; k++) out[k] = pack2(__uint_as_float(v[2 * k]), __uint_as_float(v[2 * k + 1]));
                }
                if (c == OUT_BN / 32 - 1) {
                    // everything of this accumulator is in registers: the tensor cores may have it back
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty + 8 * b);
                }
                if (row < M) {
                    bf16* dst = y + (size_t)row * n_out + n0 + c * 32;
#pragma unroll
                    for (int k = 0; k < 4; k++)
                        *reinterpret_cast<uint4*>(dst + k * 8) = make_uint4(out[4 * k], out[4 * k + 1], out[4 * k + 2], out[4 * k + 3]);
                }
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
    if (threadIdx.x == 0 && *abort_flag) atomicOr(status, 64);
}

// ---- host side ----------------------------------------------------------------------------------

// Whether this kernel takes the product (n_out: columns of y).
PLLM_EXPORT int pllm_gemm_tcgen05_supports(int M, int n_out, int K, int glu) {
    return M >= 1 && K >= 64 && K % 8 == 0 && n_out >= 64 && n_out % (glu ? 64 : 128) == 0;
}

namespace {

int g_sm_count = 0;

template <int EPI, int BN, int HD>
int launch_gemm(const void* x, const void* w, void* y, int M, int n_out, int K, const QkvEpilogue& e, int* status,
                cudaStream_t stream) {
    constexpr bool GLU = EPI == 1;
    constexpr int OUT_BN = GLU ? BN / 2 : BN;
    constexpr int EPI_SMEM = EPI == 2 ? 4 * G_EPI_BUF : 0;
    constexpr int STAGE = G_TILE_A + BN * G_BK * 2, STAGES = (G_SMEM_TILES - EPI_SMEM) / STAGE;
    CUtensorMap map_a, map_b;
    {
        const long long da[2] = {K, M}, db[2] = {K, GLU ? 2LL * n_out : n_out}, st[1] = {2LL * K};
        const int ba[2] = {G_BK, G_BM}, bb[2] = {G_BK, OUT_BN};
        if (tensor_map(x, 2, da, st, ba, true, &map_a) != 0) return PLLM_ERR_SIZE;
        if (tensor_map(w, 2, db, st, bb, true, &map_b) != 0) return PLLM_ERR_SIZE;
    }
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    const size_t smem = (size_t)STAGES * STAGE + 8 * (2 * STAGES + 4) + 16 + EPI_SMEM + 1024;
    const int n_tiles = ((M + G_BM - 1) / G_BM) * (n_out / OUT_BN);
    const dim3 grid(n_tiles < g_sm_count ? n_tiles : g_sm_count);
    cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI, BN, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(gemm_tcgen05_kernel<EPI, BN, HD>, grid, dim3(G_THREADS), smem, stream, map_a, map_b, (bf16*)y, M, n_out, K, e,
                   status);
    return launch_status();
}

}  // namespace

// x: [M, K]; w: [n_out, K], or with glu [2 n_out, K] = gate rows then up rows; y: [M, n_out]; all bfloat16.
PLLM_EXPORT int pllm_gemm_tcgen05(const void* x, const void* w, void* y, int M, int n_out, int K, int glu, int* status,
                                  cudaStream_t stream) {
    if (!pllm_gemm_tcgen05_supports(M, n_out, K, glu)) return PLLM_ERR_SIZE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) return PLLM_ERR_ALIGN;
    // tiles of 256 columns of W where the width divides into them and they still give every SM one
    const int tiles_m = (M + G_BM - 1) / G_BM;
    const int unit = glu ? 128 : 256;
    const bool wide = n_out % unit == 0 && (long long)tiles_m * (n_out / unit) >= 148;
    const QkvEpilogue none = {};
    if (glu)
        return wide ? launch_gemm<1, 256, 64>(x, w, y, M, n_out, K, none, status, stream)
                    : launch_gemm<1, 128, 64>(x, w, y, M, n_out, K, none, status, stream);
    return wide ? launch_gemm<0, 256, 64>(x, w, y, M, n_out, K, none, status, stream)
                : launch_gemm<0, 128, 64>(x, w, y, M, n_out, K, none, status, stream);
}

// Whether pllm_gemm_tcgen05_qkv takes the projection: heads of 64 or 128 values that tile the 128 (or 256)
// columns of a tile, rotated over their whole width or not at all.
PLLM_EXPORT int pllm_gemm_tcgen05_qkv_supports(int M, int K, int nh, int nkv, int hd, int rotary_dim) {
    if (hd != 64 && hd != 128) return 0;
    if (rotary_dim != 0 && rotary_dim != hd) return 0;
    if (nh <= 0 || nkv <= 0) return 0;
    // every run of columns the kernel may be asked for (q alone, or q, k and v) must be whole tiles
    return M >= 1 && K >= 64 && K % 8 == 0 && (nh * hd) % 128 == 0 && ((nh + 2 * nkv) * hd) % 128 == 0;
}

// The attention's input projection with the per-head norm, the rotation and the cache write in its
// epilogue.  x: [M, K]; w: [(nh + 2 nkv) * hd, K] = q rows, k rows, v rows; q_out: [M, nh * hd];
// k_pool / v_pool null: only q is made (and only its columns are multiplied).  Gains and tables may be null.
PLLM_EXPORT int pllm_gemm_tcgen05_qkv(const void* x, const void* w, void* q_out, const float* q_gain, const float* k_gain,
                                      float eps, const float* cos_t, const float* sin_t, int max_pos, const int* positions,
                                      const int* slots, void* k_pool, void* v_pool, int M, int K, int nh, int nkv, int hd,
                                      int page_size, int n_pages, int swizzle, int* status, cudaStream_t stream) {
    if (!pllm_gemm_tcgen05_qkv_supports(M, K, nh, nkv, hd, cos_t ? hd : 0)) return PLLM_ERR_SIZE;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)q_out | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) return PLLM_ERR_ALIGN;
    if ((cos_t == nullptr) != (sin_t == nullptr) || positions == nullptr || page_size <= 0) return PLLM_ERR_SIZE;
    if (swizzle && hd % 64) return PLLM_ERR_SIZE;     // a swizzled row is whole groups of eight 16-byte chunks
    const bool keep = k_pool != nullptr && v_pool != nullptr && slots != nullptr;
    const int n_out = (keep ? nh + 2 * nkv : nh) * hd;
    const QkvEpilogue e = {(bf16*)q_out, keep ? (bf16*)k_pool : nullptr, keep ? (bf16*)v_pool : nullptr, positions, slots,
                           q_gain, k_gain, cos_t, sin_t, eps, nh, nkv, page_size, n_pages, max_pos, swizzle};
    const int tiles_m = (M + G_BM - 1) / G_BM;
    const bool wide = n_out % 256 == 0 && (nh * hd) % 256 == 0 && (long long)tiles_m * (n_out / 256) >= 148;
    if (hd == 128)
        return wide ? launch_gemm<2, 256, 128>(x, w, nullptr, M, n_out, K, e, status, stream)
                    : launch_gemm<2, 128, 128>(x, w, nullptr, M, n_out, K, e, status, stream);
    return wide ? launch_gemm<2, 256, 64>(x, w, nullptr, M, n_out, K, e, status, stream)
                : launch_gemm<2, 128, 64>(x, w, nullptr, M, n_out, K, e, status, stream);
}

PLLM_TRACE_EXPORT(gemm_tcgen05)

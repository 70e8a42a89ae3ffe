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

}  // namespace

// map_a: x [M, K], box 64 x 128.  map_b: W [rows, K], box 64 x BN (plain) or 64 x BN/2 (GLU).
// y: [M, n_out] bfloat16; n_out = N (plain) or N / 2 (GLU, W = [gate; up] of n_out rows each).
template <int EPI, int BN>
__global__ void __launch_bounds__(G_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                    const __grid_constant__ CUtensorMap map_b,
                                                                    bf16* __restrict__ y, int M, int n_out, int K,
                                                                    int* status) {
    constexpr bool GLU = EPI == 1;
    constexpr int TILE_B = BN * G_BK * 2, STAGE = G_TILE_A + TILE_B;
    constexpr int STAGES = G_SMEM_TILES / STAGE;
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


template <int EPI, int BN>
int launch_gemm(const void* x, const void* w, void* y, int M, int n_out, int K, int* status,
                cudaStream_t stream) {
    constexpr bool GLU = EPI == 1;
    constexpr int OUT_BN = GLU ? BN / 2 : BN;
    constexpr int STAGE = G_TILE_A + BN * G_BK * 2, STAGES = G_SMEM_TILES / STAGE;
    CUtensorMap map_a, map_b;
    {
        const long long da[2] = {K, M}, db[2] = {K, GLU ? 2LL * n_out : n_out}, st[1] = {2LL * K};
        const int ba[2] = {G_BK, G_BM}, bb[2] = {G_BK, OUT_BN};
        if (tensor_map(x, 2, da, st, ba, true, &map_a) != 0) return PLLM_ERR_SIZE;
        if (tensor_map(w, 2, db, st, bb, true, &map_b) != 0) return PLLM_ERR_SIZE;
    }
    const int g_sm_count = sm_count();
    const size_t smem = (size_t)STAGES * STAGE + 8 * (2 * STAGES + 4) + 16 + 1024;
    const int n_tiles = ((M + G_BM - 1) / G_BM) * (n_out / OUT_BN);
    const dim3 grid(n_tiles < g_sm_count ? n_tiles : g_sm_count);
    cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(gemm_tcgen05_kernel<EPI, BN>, grid, dim3(G_THREADS), smem, stream, map_a, map_b, (bf16*)y, M, n_out, K, status);
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
    const bool wide = n_out % unit == 0 && (long long)tiles_m * (n_out / unit) >= sm_count();
    if (glu)
        return wide ? launch_gemm<1, 256>(x, w, y, M, n_out, K, status, stream)
                    : launch_gemm<1, 128>(x, w, y, M, n_out, K, status, stream);
    return wide ? launch_gemm<0, 256>(x, w, y, M, n_out, K, status, stream)
                : launch_gemm<0, 128>(x, w, y, M, n_out, K, status, stream);
}

PLLM_TRACE_EXPORT(gemm_tcgen05)

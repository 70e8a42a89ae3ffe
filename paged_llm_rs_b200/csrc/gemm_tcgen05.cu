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
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace {

constexpr int G_BM = 128, G_BK = 64;
constexpr int G_TILE_A = G_BM * G_BK * 2;           // 16 KB
constexpr int G_SMEM_TILES = 192 * 1024;            // what the stages may fill
constexpr int G_SPIN_LIMIT = 1 << 22;
constexpr int G_THREADS = 192;

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
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Waits until the barrier's phase `parity` is over; gives up after a bounded number of polls
// or when another thread has given up.  Returns false then.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int spin = 0; spin < G_SPIN_LIMIT; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255) == 255 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bfloat16),
// stored with the 128-byte swizzle in groups of 8 rows (1024 bytes): start address, leading
// byte offset 1 (unused with a swizzle), stride byte offset 1024, version 1, layout 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fff) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: float accumulator, bfloat16 A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t addr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(addr));
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

}  // namespace

// map_a: x [M, K], box 64 x 128.  map_b: W [rows, K], box 64 x BN (plain) or 64 x BN/2 (GLU).
// y: [M, n_out] bfloat16; n_out = N (plain) or N / 2 (GLU, W = [gate; up] of n_out rows each).
template <int GLU, int BN>
__global__ void __launch_bounds__(G_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                    const __grid_constant__ CUtensorMap map_b,
                                                                    bf16* __restrict__ y, int M, int n_out, int K,
                                                                    int* status) {
    constexpr int TILE_B = BN * G_BK * 2, STAGE = G_TILE_A + TILE_B, STAGES = G_SMEM_TILES / STAGE;
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
            pdl_wait();      // x comes from the kernel before this one
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

namespace {

struct MapKey {
    const void* ptr; int rows, cols, box_rows;
    bool operator<(const MapKey& o) const { return std::tie(ptr, rows, cols, box_rows) < std::tie(o.ptr, o.rows, o.cols, o.box_rows); }
};
std::map<MapKey, CUtensorMap> g_maps;
std::mutex g_maps_lock;

// A [rows, cols] bfloat16 row-major matrix cut into boxes of box_rows x 64 with the 128-byte swizzle.
int tensor_map(const void* ptr, int rows, int cols, int box_rows, CUtensorMap* out) {
    std::lock_guard<std::mutex> hold(g_maps_lock);
    const MapKey key{ptr, rows, cols, box_rows};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)G_BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    // the driver's encoder is looked up at run time: the library then loads on a machine without a
    // driver too (where only its host-side functions are used)
    typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult found;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) != cudaSuccess || fn == nullptr)
            return -1;
        encode = (EncodeFn)fn;
    }
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)r;
    if (g_maps.size() > 4096) g_maps.clear();     // activations come and go; weights come back
    g_maps[key] = *out;
    return 0;
}

}  // namespace

// Whether this kernel takes the product (n_out: columns of y).
PLLM_EXPORT int pllm_gemm_tcgen05_supports(int M, int n_out, int K, int glu) {
    return M >= 1 && K >= 64 && K % 8 == 0 && n_out >= 64 && n_out % (glu ? 64 : 128) == 0;
}

namespace {

int g_sm_count = 0;

template <int GLU, int BN>
int launch_gemm(const void* x, const void* w, void* y, int M, int n_out, int K, int* status, cudaStream_t stream) {
    constexpr int OUT_BN = GLU ? BN / 2 : BN;
    constexpr int STAGE = G_TILE_A + BN * G_BK * 2, STAGES = G_SMEM_TILES / STAGE;
    CUtensorMap map_a, map_b;
    if (tensor_map(x, M, K, G_BM, &map_a) != 0) return PLLM_ERR_SIZE;
    if (tensor_map(w, GLU ? 2 * n_out : n_out, K, OUT_BN, &map_b) != 0) return PLLM_ERR_SIZE;
    if (g_sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    const size_t smem = (size_t)STAGES * STAGE + 8 * (2 * STAGES + 4) + 16 + 1024;
    const int n_tiles = ((M + G_BM - 1) / G_BM) * (n_out / OUT_BN);
    const dim3 grid(n_tiles < g_sm_count ? n_tiles : g_sm_count);
    cudaFuncSetAttribute(gemm_tcgen05_kernel<GLU, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(gemm_tcgen05_kernel<GLU, BN>, grid, dim3(G_THREADS), smem, stream, map_a, map_b, (bf16*)y, M, n_out, K, status);
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
    if (glu) return wide ? launch_gemm<1, 256>(x, w, y, M, n_out, K, status, stream) : launch_gemm<1, 128>(x, w, y, M, n_out, K, status, stream);
    return wide ? launch_gemm<0, 256>(x, w, y, M, n_out, K, status, stream) : launch_gemm<0, 128>(x, w, y, M, n_out, K, status, stream);
}

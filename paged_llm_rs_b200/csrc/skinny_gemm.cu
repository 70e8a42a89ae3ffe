// y[M, N] = x[M, K] . W[N, K]^T for few rows (M <= 64, a decode step) in
// bfloat16 with float accumulation: a weight-streaming kernel, bound by the bytes
// of W.  Where the reference calls a library product for every projection
// (crates/pagedllm/src/model/layers.rs:27-35), a library kernel chosen for large
// products spends 6 to 10 microseconds on each of these, several times what the
// bytes take; this kernel is for exactly that shape.
//
// Each warp owns 8 * NT rows of W and a slice of K.  Every lane reads 16
// contiguous bytes of a W row straight from global memory into registers (no
// shared memory, streaming loads) and 16 bytes of two x rows through L1, and
// feeds mma.sync.m16n8k16 with x as the A operand (rows of the step, padded to
// 16) and W as the B operand.  The tensor core sums over k in any order, so the
// k indices inside a block of 32 are dealt to the lanes as the 16-byte loads
// deliver them: lane t (mod 4) holds k = 8t .. 8t+7 of both operands.
// The warps of a CTA split K; their partial sums meet in shared memory.
//
// One thing a decode step does after a product is folded in, because at a few rows
// every kernel costs its launch and a round trip through memory, not its arithmetic:
//   EPI = 1: W is [gate rows | up rows] of a gated feed-forward and y = silu(g) * u
//     (crates/pagedllm/src/model/layers.rs:93-99): a CTA takes the same columns
//     of both halves, so the activation needs neither a pass nor a buffer.
#include "common.cuh"

#ifndef PLLM_SKINNY_EARLY
#define PLLM_SKINNY_EARLY 1
#endif

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
// x comes from the kernel before this one, which may still run while this kernel's CTAs take their
// places: a load from L2 after the wait, never the read-only path (L1 may hold the line as an
// earlier kernel on this SM saw it).
__device__ __forceinline__ uint4 ld_cached16(const void* p) {
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p) : "memory");
    return r;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int MT, int NT, int EPI, typename OutT>
__global__ void __launch_bounds__(16 * 32, 1) skinny_gemm_kernel(const bf16* x, const bf16* __restrict__ w,
                                                                 OutT* __restrict__ y, int M, int N, int K) {
    static_assert(!EPI || NT % 2 == 0, "the gated epilogue pairs tiles of gate and up");
    // k blocks of 32 whose loads are issued together
    constexpr int U = MT == 1 ? 4 : (MT == 2 ? 2 : 1);
    constexpr int ROWS = MT * 16, COLS = NT * 8, OUT_COLS = EPI ? COLS / 2 : COLS;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, ks_count = blockDim.x >> 5;
    const int n0 = blockIdx.x * OUT_COLS;
    const int k_per = K / ks_count;
    const int k_begin = warp * k_per, k_end = k_begin + k_per;
    const int r = lane >> 2, t = lane & 3;

    float acc[MT][NT][4];
#pragma unroll
    for (int a = 0; a < MT; a++)
#pragma unroll
        for (int b = 0; b < NT; b++) acc[a][b][0] = acc[a][b][1] = acc[a][b][2] = acc[a][b][3] = 0.f;

    const bf16* wrow[NT];
#pragma unroll
    for (int b = 0; b < NT; b++) {
        // gated: the first half of the tiles are gate rows, the second the same columns of up
        const int row = (EPI && b >= NT / 2) ? N + n0 + (b - NT / 2) * 8 + r : n0 + b * 8 + r;
        wrow[b] = w + (size_t)row * K + t * 8;
    }
    const bf16* xrow[MT][2];
    bool xok[MT][2];
#pragma unroll
    for (int a = 0; a < MT; a++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = a * 16 + h * 8 + r;
            xok[a][h] = m < M;
            xrow[a][h] = x + (size_t)(xok[a][h] ? m : 0) * K + t * 8;
        }
    extern __shared__ float red[];  // [warps][MT*16][NT*8]

    for (int kb = k_begin; kb < k_end; kb += 32 * U) {
        // every load of the group is issued before the first is used: one trip to memory, not U
        uint4 wf[U][NT], xf[U][MT][2];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int b = 0; b < NT; b++)
                if (kb + 32 * u < k_end) wf[u][b] = ld_stream16(wrow[b] + kb + 32 * u);
        // The weights do not depend on the kernel before this one; x does.
        if (kb == k_begin) { if (PLLM_SKINNY_EARLY) pdl_launch_dependents(); pdl_wait(KID_GEMM); }
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int a = 0; a < MT; a++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    xf[u][a][h] = make_uint4(0, 0, 0, 0);
                    if (xok[a][h] && kb + 32 * u < k_end) xf[u][a][h] = ld_cached16(xrow[a][h] + kb + 32 * u);
                }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (kb + 32 * u >= k_end) break;
#pragma unroll
            for (int a = 0; a < MT; a++) {
                const uint4 xa = xf[u][a][0], xb = xf[u][a][1];
#pragma unroll
                for (int b = 0; b < NT; b++) {
                    mma16816(acc[a][b], xa.x, xb.x, xa.y, xb.y, wf[u][b].x, wf[u][b].y);
                    mma16816(acc[a][b], xa.z, xb.z, xa.w, xb.w, wf[u][b].z, wf[u][b].w);
                }
            }
        }
    }

    if (!PLLM_SKINNY_EARLY) pdl_launch_dependents();   // the weights are read: the next kernel may start on its own
    // ---- the warps' partial sums over their slices of K meet in shared memory ---------------
    if (ks_count > 1 || EPI) {
        float* mine = red + (size_t)warp * ROWS * COLS;
#pragma unroll
        for (int a = 0; a < MT; a++)
#pragma unroll
            for (int b = 0; b < NT; b++) {
                const int c = b * 8 + t * 2;
                mine[(a * 16 + r) * COLS + c] = acc[a][b][0];
                mine[(a * 16 + r) * COLS + c + 1] = acc[a][b][1];
                mine[(a * 16 + 8 + r) * COLS + c] = acc[a][b][2];
                mine[(a * 16 + 8 + r) * COLS + c + 1] = acc[a][b][3];
            }
        __syncthreads();
        for (int idx = threadIdx.x; idx < ROWS * OUT_COLS; idx += blockDim.x) {
            const int m = idx / OUT_COLS, c = idx % OUT_COLS;
            if (m >= M) continue;
            float s = 0.f;
            for (int wi = 0; wi < ks_count; wi++) s += red[(size_t)wi * ROWS * COLS + m * COLS + c];  // fixed order
            if (EPI) {
                float u = 0.f;
                for (int wi = 0; wi < ks_count; wi++) u += red[(size_t)wi * ROWS * COLS + m * COLS + OUT_COLS + c];
                // gate and up are rounded as a product of their own would leave them
                const float g = __bfloat162float(__float2bfloat16_rn(s));
                u = __bfloat162float(__float2bfloat16_rn(u));
                s = g / (1.0f + expf(-g)) * u;
            }
            y[(size_t)m * N + n0 + c] = from_f32<OutT>(s);
        }
    } else {
#pragma unroll
        for (int a = 0; a < MT; a++)
#pragma unroll
            for (int b = 0; b < NT; b++) {
                const int c = n0 + b * 8 + t * 2;
                const int m0 = a * 16 + r, m1 = m0 + 8;
                if (m0 < M) { y[(size_t)m0 * N + c] = from_f32<OutT>(acc[a][b][0]); y[(size_t)m0 * N + c + 1] = from_f32<OutT>(acc[a][b][1]); }
                if (m1 < M) { y[(size_t)m1 * N + c] = from_f32<OutT>(acc[a][b][2]); y[(size_t)m1 * N + c + 1] = from_f32<OutT>(acc[a][b][3]); }
            }
    }
}

// For tuning runs: a number of warps a CTA to use instead of the heuristic's (0: the heuristic), and
// likewise the number of 8-row tiles of W a CTA takes (1, 2 or 4).
static int g_skinny_warps_override = 0, g_skinny_nt_override = 0;
PLLM_EXPORT int pllm_skinny_gemm_set_warps(int warps) {
    const int was = g_skinny_warps_override;
    g_skinny_warps_override = warps;
    return was;
}
PLLM_EXPORT int pllm_skinny_gemm_set_tiles(int nt) {
    const int was = g_skinny_nt_override;
    g_skinny_nt_override = nt;
    return was;
}

// Whether this kernel takes the product; the library takes the rest.
PLLM_EXPORT int pllm_skinny_gemm_supports(int M, int N, int K) {
    return M >= 1 && M <= 64 && N % 16 == 0 && K % 128 == 0 && N >= 16 && K >= 128;
}
// The same for the form with the gate after (N: columns of y).
PLLM_EXPORT int pllm_skinny_gemm_glu_supports(int M, int N, int K) {
    return M >= 1 && M <= 16 && N % 16 == 0 && K % 128 == 0 && N >= 16 && K >= 128;
}

template <int MT, int NT, int EPI, typename OutT>
static int launch_skinny(const void* x, const void* w, void* y, int M, int N, int K, int warps, cudaStream_t stream) {
    const size_t smem = (warps > 1 || EPI) ? (size_t)warps * MT * 16 * NT * 8 * sizeof(float) : 0;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(skinny_gemm_kernel<MT, NT, EPI, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    constexpr int out_cols = EPI ? 4 * NT : 8 * NT;
    launch_chained(skinny_gemm_kernel<MT, NT, EPI, OutT>, dim3(N / out_cols), dim3(warps * 32), smem, stream,
                   (const bf16*)x, (const bf16*)w, (OutT*)y, M, N, K);
    return launch_status();
}

template <int NT, typename OutT>
static int pick_mt(const void* x, const void* w, void* y, int M, int N, int K, int warps, cudaStream_t s) {
    if (M <= 16) return launch_skinny<1, NT, 0, OutT>(x, w, y, M, N, K, warps, s);
    if (M <= 32) return launch_skinny<2, NT, 0, OutT>(x, w, y, M, N, K, warps, s);
    if (M <= 48) return launch_skinny<3, NT, 0, OutT>(x, w, y, M, N, K, warps, s);
    return launch_skinny<4, NT, 0, OutT>(x, w, y, M, N, K, warps, s);
}

// K is split over the warps of a CTA.  A warp's loads of ``slice`` values of k are all
// issued before the first is used, so a slice costs one trip to memory: as many warps as
// give each such a slice (at most 16, and K must divide evenly into slices that are
// multiples of 32), unless the launch would then exceed what the SMs hold at once
// several times over.
// (warps_an_sm: how many warps the launch may have for every SM there is)
static int pick_warps(int K, int ctas, int slice, int warps_an_sm = 64, int max_warps = 16) {
    int warps = 1;
    // (2, 4, 8 or 16: 10 warps of 128 registers leave an SM room for one CTA where 8 leave it room for two)
    for (int wv = 2; wv <= max_warps; wv *= 2)
        if (K % (wv * 32) == 0 && K / wv >= slice && (long long)ctas * wv <= (long long)sm_count() * warps_an_sm) warps = wv;
    if (g_skinny_warps_override > 0 && g_skinny_warps_override <= 16 && K % (g_skinny_warps_override * 32) == 0)
        warps = g_skinny_warps_override;
    return warps;
}

// x: [M, K]; w: [N, K]; y: [M, N] bfloat16 (out_f32 0) or float (out_f32 1).
PLLM_EXPORT int pllm_skinny_gemm(const void* x, const void* w, void* y, int M, int N, int K, int out_f32,
                                 cudaStream_t stream) {
    if (!pllm_skinny_gemm_supports(M, N, K)) return PLLM_ERR_SIZE;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return PLLM_ERR_ALIGN;
    // More than 16 rows: tiles of 16 rows of W while that still gives every SM several CTAs, else of 8.
    const int sms = sm_count();
    int nt = (N / 16 >= 2 * sms || (K >= 4096 && N / 16 >= sms)) ? 2 : 1;
    int warps_an_sm = 64;
    int max_warps = 16;
    if (M <= 16) {
        // Up to 16 rows (a decode step).  Every CTA reads all of x from L2, and a wider tile of W does it for more
        // rows of W; but a CTA of 32-row tiles holds 128 registers a thread (with 16 warps it would fill an SM's
        // register file alone, and the kernels around it could not take their places beside it) and streams 64 K
        // bytes of W.  The rule below was decided by the decode step's time with ONE product's tiles and warps
        // changed at a time, at the 0.6B, 8B and 32B shapes (timed back to back on their own the same products
        // rank otherwise: a 32-row tile with 16 warps wins there, and loses 4 to 17 us a layer in the step):
        //   tiles of 32 rows and up to 8 warps  where that gives every SM a CTA and rows are at most 4096 long
        //                                        (6144 x 4096: 5 us a layer better than 16 rows with 16 warps);
        //   else tiles of 16 rows               where that gives every SM a CTA, with 16 warps where the rows are
        //                                        at least as long as there are rows (the o and down products:
        //                                        4096 x 12288 17 us better than 32 rows, 5120 x 25600 35 us), with
        //                                        8 where there are more rows than they are long (10240 x 5120: 13 us
        //                                        better than with 16, 30 better than 32-row tiles with 4);
        //   else tiles of 8 rows with 16 warps  (1024 x 2048, 1024 x 3072: the best of eight).
        nt = 1;
        if (N % 32 == 0 && N / 32 >= sms && K <= 4096) { nt = 4; max_warps = 8; warps_an_sm = 16; }
        else if (N % 16 == 0 && N / 16 >= sms) { nt = 2; max_warps = N > K ? 8 : 16; }
    }
    if (g_skinny_nt_override && N % (8 * g_skinny_nt_override) == 0 && (g_skinny_nt_override < 4 || M <= 16)) nt = g_skinny_nt_override;
    const int warps = pick_warps(K, N / (8 * nt), 128, warps_an_sm, max_warps);
    if (nt == 4)
        return out_f32 ? launch_skinny<1, 4, 0, float>(x, w, y, M, N, K, warps, stream)
                       : launch_skinny<1, 4, 0, bf16>(x, w, y, M, N, K, warps, stream);
    if (out_f32)
        return nt == 2 ? pick_mt<2, float>(x, w, y, M, N, K, warps, stream) : pick_mt<1, float>(x, w, y, M, N, K, warps, stream);
    return nt == 2 ? pick_mt<2, bf16>(x, w, y, M, N, K, warps, stream) : pick_mt<1, bf16>(x, w, y, M, N, K, warps, stream);
}

// w is [2N, K], gate rows then up rows, and y[M, N] = silu(x Wg^T) * (x Wu^T); up to 16 rows, all bfloat16.
PLLM_EXPORT int pllm_skinny_gemm_glu(const void* x, const void* w, void* y, int M, int N, int K, cudaStream_t stream) {
    if (!pllm_skinny_gemm_glu_supports(M, N, K)) return PLLM_ERR_SIZE;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return PLLM_ERR_ALIGN;
    // Tiles of 16 columns of y (16 gate rows and 16 up rows of W) where that gives four fifths of the SMs a CTA and
    // either the rows are long or the tiles are few enough to be in place at once; else of 8.  Measured at 8 rows,
    // microseconds with tiles of 8 / of 16: 3072 x 1024 4.6 / 3.6, 12288 x 4096 38.6 / 36.6, 25600 x 5120 91.3 / 82.6,
    // 9728 x 2560 22.2 / 23.6 (the one that stays with 8).
    const int sms = sm_count();
    int nt = (N % 16 == 0 && N / 16 >= sms * 4 / 5 && (K >= 4096 || N / 16 <= 2 * sms)) ? 4 : 2;
    if ((g_skinny_nt_override == 4 && N % 16 == 0) || g_skinny_nt_override == 2) nt = g_skinny_nt_override;
    if (nt == 4) {
        const int warps = pick_warps(K, N / 16, 128);
        return launch_skinny<1, 4, 1, bf16>(x, w, y, M, N, K, warps, stream);
    }
    const int warps = pick_warps(K, N / 8, 128);
    return launch_skinny<1, 2, 1, bf16>(x, w, y, M, N, K, warps, stream);
}

PLLM_TRACE_EXPORT(skinny_gemm)

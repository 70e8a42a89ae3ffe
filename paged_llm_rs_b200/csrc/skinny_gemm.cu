// y[M, N] = act(x)[M, K] . W[N, K]^T for few rows (M <= 64, a decode step) in
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
// act = 1: the A operand is silu(g) * u formed on the fly from x = [g | u]
// ([M, 2K]), the gated feed-forward's activation
// (crates/pagedllm/src/model/layers.rs:93-99), so the activation needs no pass
// of its own.
#include "common.cuh"

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ uint4 ld_cached16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t silu_mul2(uint32_t g, uint32_t u) {
    // two bfloat16 in each word: silu(g) * u in float, rounded once
    const float g0 = __uint_as_float(g << 16), g1 = __uint_as_float(g & 0xffff0000u);
    const float u0 = __uint_as_float(u << 16), u1 = __uint_as_float(u & 0xffff0000u);
    __nv_bfloat162 h = __floats2bfloat162_rn(g0 / (1.0f + expf(-g0)) * u0, g1 / (1.0f + expf(-g1)) * u1);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int MT, int NT, int ACT, typename OutT>
__global__ void __launch_bounds__(512) skinny_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          OutT* __restrict__ y, int M, int N, int K, int ldx) {
    constexpr int U = MT == 1 ? 4 : (MT == 2 ? 2 : 1);  // k blocks of 32 whose loads are issued together
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, ks_count = blockDim.x >> 5;
    const int n0 = blockIdx.x * (8 * NT);
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
    for (int b = 0; b < NT; b++) wrow[b] = w + (size_t)(n0 + b * 8 + r) * K + t * 8;
    const bf16* xrow[MT][2];
    bool xok[MT][2];
#pragma unroll
    for (int a = 0; a < MT; a++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int m = a * 16 + h * 8 + r;
            xok[a][h] = m < M;
            xrow[a][h] = x + (size_t)(xok[a][h] ? m : 0) * ldx + t * 8;
        }

    for (int kb = k_begin; kb < k_end; kb += 32 * U) {
        // every load of the group is issued before the first is used: one trip to memory, not U
        uint4 wf[U][NT], xf[U][MT][2];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int b = 0; b < NT; b++)
                if (kb + 32 * u < k_end) wf[u][b] = ld_stream16(wrow[b] + kb + 32 * u);
        // The weights do not depend on the kernel before this one; x does.
        if (kb == k_begin) pdl_wait();
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
            const int k = kb + 32 * u;
#pragma unroll
            for (int a = 0; a < MT; a++) {
                uint4 xa = xf[u][a][0], xb = xf[u][a][1];
                if (ACT == 1) {
                    uint4 ua = make_uint4(0, 0, 0, 0), ub = make_uint4(0, 0, 0, 0);
                    if (xok[a][0]) ua = ld_cached16(xrow[a][0] + K + k);
                    if (xok[a][1]) ub = ld_cached16(xrow[a][1] + K + k);
                    xa = make_uint4(silu_mul2(xa.x, ua.x), silu_mul2(xa.y, ua.y), silu_mul2(xa.z, ua.z), silu_mul2(xa.w, ua.w));
                    xb = make_uint4(silu_mul2(xb.x, ub.x), silu_mul2(xb.y, ub.y), silu_mul2(xb.z, ub.z), silu_mul2(xb.w, ub.w));
                }
#pragma unroll
                for (int b = 0; b < NT; b++) {
                    mma16816(acc[a][b], xa.x, xb.x, xa.y, xb.y, wf[u][b].x, wf[u][b].y);
                    mma16816(acc[a][b], xa.z, xb.z, xa.w, xb.w, wf[u][b].z, wf[u][b].w);
                }
            }
        }
    }

    pdl_launch_dependents();   // the weights are read: the next kernel may start on its own
    // ---- the warps' partial sums over their slices of K meet in shared memory ---------------
    extern __shared__ float red[];  // [warps][MT*16][NT*8]
    constexpr int ROWS = MT * 16, COLS = NT * 8;
    if (ks_count > 1) {
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
        for (int idx = threadIdx.x; idx < ROWS * COLS; idx += blockDim.x) {
            const int m = idx / COLS, c = idx % COLS;
            if (m >= M) continue;
            float s = 0.f;
            for (int wi = 0; wi < ks_count; wi++) s += red[(size_t)wi * ROWS * COLS + idx];  // fixed order
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

// For tuning runs: a number of warps a CTA to use instead of the heuristic's (0: the heuristic).
static int g_skinny_warps_override = 0;
PLLM_EXPORT int pllm_skinny_gemm_set_warps(int warps) {
    const int was = g_skinny_warps_override;
    g_skinny_warps_override = warps;
    return was;
}

// Whether this kernel takes the product; the library takes the rest.
PLLM_EXPORT int pllm_skinny_gemm_supports(int M, int N, int K) {
    return M >= 1 && M <= 64 && N % 16 == 0 && K % 128 == 0 && N >= 16 && K >= 128;
}

template <int MT, int NT, int ACT, typename OutT>
static int launch_skinny(const void* x, const void* w, void* y, int M, int N, int K, int ldx, int warps,
                         cudaStream_t stream) {
    const size_t smem = warps > 1 ? (size_t)warps * MT * 16 * NT * 8 * sizeof(float) : 0;
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(skinny_gemm_kernel<MT, NT, ACT, OutT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_chained(skinny_gemm_kernel<MT, NT, ACT, OutT>, dim3(N / (8 * NT)), dim3(warps * 32), smem, stream,
                   (const bf16*)x, (const bf16*)w, (OutT*)y, M, N, K, ldx);
    return launch_status();
}

template <int NT, int ACT, typename OutT>
static int pick_mt(const void* x, const void* w, void* y, int M, int N, int K, int ldx, int warps, cudaStream_t s) {
    if (M <= 16) return launch_skinny<1, NT, ACT, OutT>(x, w, y, M, N, K, ldx, warps, s);
    if (M <= 32) return launch_skinny<2, NT, ACT, OutT>(x, w, y, M, N, K, ldx, warps, s);
    if (M <= 48) return launch_skinny<3, NT, ACT, OutT>(x, w, y, M, N, K, ldx, warps, s);
    return launch_skinny<4, NT, ACT, OutT>(x, w, y, M, N, K, ldx, warps, s);
}

// x: [M, K] (act 0) or [M, 2K] (act 1: silu(x[:, :K]) * x[:, K:]); w: [N, K]; y: [M, N]
// bfloat16 (out_f32 0) or float (out_f32 1).
PLLM_EXPORT int pllm_skinny_gemm(const void* x, const void* w, void* y, int M, int N, int K, int act, int out_f32,
                                 cudaStream_t stream) {
    if (!pllm_skinny_gemm_supports(M, N, K) || act < 0 || act > 1) return PLLM_ERR_SIZE;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return PLLM_ERR_ALIGN;
    const int ldx = act ? 2 * K : K;
    // Tiles of 16 rows of W while that still gives every SM several CTAs, else of 8;
    // K is split over the warps of a CTA in slices of at least 128.
    const int nt = (N / 16 >= 2 * 148) ? 2 : 1;
    const int ctas = N / (8 * nt);
    // A warp's loads of 128 values of k are all issued before the first is used, so a slice
    // of 128 costs one trip to memory: as many warps as give each such a slice (at most 16,
    // and K must divide evenly into slices that are multiples of 32), unless the launch
    // would then exceed what the SMs hold at once several times over.
    int warps = 1;
    for (int wv = 2; wv <= 16; wv++)
        if (K % (wv * 32) == 0 && K / wv >= 128 && (long long)ctas * wv <= 148LL * 64) warps = wv;
    if (g_skinny_warps_override > 0 && K % (g_skinny_warps_override * 32) == 0) warps = g_skinny_warps_override;
    if (out_f32) {
        if (act) return PLLM_ERR_SIZE;
        return nt == 2 ? pick_mt<2, 0, float>(x, w, y, M, N, K, ldx, warps, stream)
                       : pick_mt<1, 0, float>(x, w, y, M, N, K, ldx, warps, stream);
    }
    if (act)
        return nt == 2 ? pick_mt<2, 1, bf16>(x, w, y, M, N, K, ldx, warps, stream)
                       : pick_mt<1, 1, bf16>(x, w, y, M, N, K, ldx, warps, stream);
    return nt == 2 ? pick_mt<2, 0, bf16>(x, w, y, M, N, K, ldx, warps, stream)
                   : pick_mt<1, 0, bf16>(x, w, y, M, N, K, ldx, warps, stream);
}

// Shared helpers of the sm_100a kernels: element conversion, vector access,
// warp and block reductions, and the return codes of the C entry points.
//
// Every kernel is a template over the element type (float for the true 32-bit
// path, __nv_bfloat16 for serving) and does its arithmetic in float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#define PLLM_EXPORT extern "C" __attribute__((visibility("default")))

// Return codes of the C entry points.  0 is success; positive values are
// cudaError_t from the launch; negative values are refusals of the arguments.
enum : int {
    PLLM_OK = 0,
    PLLM_ERR_DTYPE = -1,      // dtype code not 0 (float32) or 1 (bfloat16)
    PLLM_ERR_SIZE = -2,       // a size the kernel does not take
    PLLM_ERR_ALIGN = -3,      // a pointer or stride that is not aligned as required
    PLLM_ERR_LIMIT = -4,      // a size beyond a stated maximum
};

enum : int { PLLM_F32 = 0, PLLM_BF16 = 1 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    return warp_sum(r);
}

// 16-byte vectors of elements: 4 floats or 8 bfloat16.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    float4 raw;
    __device__ __forceinline__ void load(const float* p) { raw = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ void store(float* p) const { *reinterpret_cast<float4*>(p) = raw; }
    __device__ __forceinline__ void unpack(float* f) const { f[0] = raw.x; f[1] = raw.y; f[2] = raw.z; f[3] = raw.w; }
    __device__ __forceinline__ void pack(const float* f) { raw = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    uint4 raw;
    __device__ __forceinline__ void load(const bf16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void store(bf16* p) const { *reinterpret_cast<uint4*>(p) = raw; }
    __device__ __forceinline__ void unpack(float* f) const {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            // a bfloat16 is the upper half of a float
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ __forceinline__ void pack(const float* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        raw = make_uint4(w[0], w[1], w[2], w[3]);
    }
};

static inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? PLLM_OK : (int)e;
}

// Streaming multiprocessors of the current device (asked once; grids are sized by it).
static inline int sm_count() {
    static int count = 0;
    if (count <= 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            return 148;       // (a B200; asked again next time)
        count = n;
    }
    return count;
}

// ---- programmatic dependent launch -------------------------------------------------------
// A decode step is a chain of a few hundred short kernels, each waiting for the one
// before it.  Launched with the programmatic-serialization attribute, a kernel's CTAs
// may take their places on the SMs while the kernel before it is still running; they
// call pdl_wait() before they touch anything an earlier kernel wrote (it returns
// when every earlier kernel of the stream has finished and its writes are visible),
// and pdl_launch_dependents() lets the kernel after them do the same.  What does not
// depend on earlier kernels (reading weights) may come before the wait.
// One rule follows for every kernel here: a pointer to data that a kernel shortly before it in
// the stream writes (activations, partial results, this step's cache rows) is never
// `const __restrict__` and never read with __ldg.  Those make the compiler use the SM's
// read-only cache, which is only right for data that does not change while the kernel is
// resident, and a kernel launched early is resident while its input is still being written:
// it can then hit a line that an older kernel left on the same SM at the same (recycled)
// address.  It showed as wrong tokens with a tiny model, whose kernels are all resident
// at once.  Weights, tables and the host's step buffer may use the read-only path.
// Without the attribute both calls do nothing.
#ifndef PLLM_TRACE
__device__ __forceinline__ void pdl_wait(int kernel_id = 0, bool this_thread = false) { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
#define PLLM_TRACE_EXPORT(file)
#else
// A build for timelines (-DPLLM_TRACE=1): thread 0 of block (0, 0) of every kernel stamps the
// global timer before and after its wait for the kernel before it, with the kernel's id, into a
// buffer of this source file.  The time between two kernels' "after" stamps is what the earlier
// one costs in the chain; "before" shows how early a kernel's CTAs were in place.
#define PLLM_TRACE_SLOTS 8192
static __device__ unsigned long long g_trace[PLLM_TRACE_SLOTS * 3];
static __device__ unsigned int g_trace_n;
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}
// (this_thread: the caller is the one thread of the kernel's first CTA that is to stamp, in kernels
// whose thread 0 does not wait)
__device__ __forceinline__ void pdl_wait(int kernel_id = 0, bool this_thread = false) {
    const bool me = this_thread ? (blockIdx.x | blockIdx.y | blockIdx.z) == 0
                                : (threadIdx.x | threadIdx.y | blockIdx.x | blockIdx.y | blockIdx.z) == 0;
    const unsigned long long t0 = me ? global_ns() : 0;
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    if (me) {
        const unsigned int i = atomicAdd(&g_trace_n, 1u);
        if (i < PLLM_TRACE_SLOTS) { g_trace[3 * i] = (unsigned long long)kernel_id; g_trace[3 * i + 1] = t0; g_trace[3 * i + 2] = global_ns(); }
    }
}
// Copies the stamps out (3 x 64-bit each: id, before, after), empties the buffer, returns the count.
#define PLLM_TRACE_EXPORT(file)                                                                              \
    PLLM_EXPORT int pllm_trace_read_##file(unsigned long long* out, int max_records) {                       \
        unsigned int n = 0, zero = 0;                                                                        \
        cudaDeviceSynchronize();                                                                             \
        cudaMemcpyFromSymbol(&n, g_trace_n, sizeof(n));                                                      \
        if (n > PLLM_TRACE_SLOTS) n = PLLM_TRACE_SLOTS;                                                      \
        if ((int)n > max_records) n = max_records;                                                           \
        if (n) cudaMemcpyFromSymbol(out, g_trace, (size_t)n * 3 * sizeof(unsigned long long));               \
        cudaMemcpyToSymbol(g_trace_n, &zero, sizeof(zero));                                                  \
        return (int)n;                                                                                       \
    }
#endif
// Kernel ids of the timeline.
enum : int { KID_EMBED = 1, KID_RMSNORM, KID_SWIGLU, KID_QK, KID_ATT_GENERIC, KID_ATT_REDUCE, KID_ATT_MMA, KID_ATT_TMA,
             KID_GEMM, KID_SAMPLE_PART, KID_SAMPLE_FINAL, KID_GEMM_TC, KID_ATT_TC };
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }

extern int pllm_pdl_enabled;  // defined in elementwise.cu; set through pllm_set_pdl

template <typename... KArgs, typename... Args>
static inline void launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pllm_pdl_enabled ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same with the CTAs of `cluster_y` consecutive blockIdx.y in one thread-block cluster (they
// run at the same time on neighbouring SMs and may read one another's shared memory).
template <typename... KArgs, typename... Args>
static inline void launch_chained_cluster_y(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                            int cluster_y, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = (unsigned)cluster_y;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pllm_pdl_enabled ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define PLLM_DISPATCH_DTYPE(dtype, ...)                         \
    do {                                                        \
        if ((dtype) == PLLM_F32) { typedef float T; __VA_ARGS__; } \
        else if ((dtype) == PLLM_BF16) { typedef bf16 T; __VA_ARGS__; } \
        else return PLLM_ERR_DTYPE;                             \
    } while (0)

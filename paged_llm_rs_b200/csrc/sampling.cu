// Choosing the next token on the device: greedy argmax and a temperature draw.
//
// Greedy takes the first maximum (crates/pagedllm/src/sampler.rs:186-194).  The
// temperature draw scales logits by 1/T, forms exp(l - max) in float and picks
// the token where the running sum first reaches u * total (sampler.rs:123-183),
// u being the request's own uniform number, made on the host by its splitmix64
// generator.  The reference walks the tokens in order of falling probability;
// this kernel walks them in order of their ids, which gives every token the same
// probability and needs no sort.  (Requests with top-k or top-p go through the
// host sampler, which keeps the reference's order.)
//
// Two launches.  The first cuts every row into chunks of 4096 logits, one CTA
// each, and writes per chunk (max, index of the first max, sum of exp((l - max)/T))
// to scratch memory.  The second, one CTA per row, combines the chunks in their
// order, finds the chunk the draw falls into and walks that chunk alone.  All
// sums are formed in a fixed order, so a draw does not depend on timing.
#include "common.cuh"

#define SAMPLE_CHUNK 4096
#define SAMPLE_THREADS 256
#define SAMPLE_PER_THREAD (SAMPLE_CHUNK / SAMPLE_THREADS)

__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// scratch: [rows][chunks][4] floats = (max, index as int bits, sum, unused)
__global__ void sample_partial_kernel(const float* logits, int vocab, long long row_stride,
                                      const float* __restrict__ temperature, float* __restrict__ scratch) {
    __shared__ float s_v[SAMPLE_THREADS / 32];
    __shared__ int s_i[SAMPLE_THREADS / 32];
    __shared__ float s_sum[SAMPLE_THREADS / 32];
    __shared__ float s_max;
    pdl_launch_dependents();
    pdl_wait(KID_SAMPLE_PART);
    const int row = blockIdx.y, chunk = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* l = logits + (size_t)row * row_stride;
    const int base = chunk * SAMPLE_CHUNK;
    float vals[SAMPLE_PER_THREAD];
    float best = -CUDART_INF_F;
    int arg = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < SAMPLE_PER_THREAD; j++) {
        const int i = base + j * SAMPLE_THREADS + tid;   // neighbouring threads read neighbouring logits
        vals[j] = i < vocab ? l[i] : -CUDART_INF_F;
        if (i < vocab && (arg == 0x7fffffff || vals[j] > best)) { best = vals[j]; arg = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_merge(best, arg, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, arg, o));
    if (lane == 0) { s_v[warp] = best; s_i[warp] = arg; }
    __syncthreads();
    if (warp == 0) {
        best = lane < SAMPLE_THREADS / 32 ? s_v[lane] : -CUDART_INF_F;
        arg = lane < SAMPLE_THREADS / 32 ? s_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            argmax_merge(best, arg, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, arg, o));
        if (lane == 0) {
            s_max = best;
            float* out = scratch + ((size_t)row * gridDim.x + chunk) * 4;
            out[0] = best;
            out[1] = __int_as_float(arg);
        }
    }
    __syncthreads();
    const float temp = temperature[row];
    if (!(temp > 0.f)) return;
    const float inv = 1.0f / temp, top = s_max * inv;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < SAMPLE_PER_THREAD; j++)
        if (base + j * SAMPLE_THREADS + tid < vocab) sum += expf(vals[j] * inv - top);
    sum = warp_sum(sum);
    if (lane == 0) s_sum[warp] = sum;
    __syncthreads();
    if (tid == 0) {
        float total = 0.f;
        for (int k = 0; k < SAMPLE_THREADS / 32; k++) total += s_sum[k];
        scratch[((size_t)row * gridDim.x + chunk) * 4 + 2] = total;
    }
}

__global__ void sample_final_kernel(const float* logits, int vocab, long long row_stride, int chunks,
                                    const float* __restrict__ temperature, const float* __restrict__ uniform,
                                    const float* scratch, int* __restrict__ tokens) {
    __shared__ float s_v[SAMPLE_THREADS / 32];
    __shared__ int s_i[SAMPLE_THREADS / 32];
    __shared__ float s_scan[SAMPLE_THREADS];
    __shared__ float s_max, s_before, s_point;
    __shared__ int s_arg, s_chunk, s_owner;
    pdl_launch_dependents();
    pdl_wait(KID_SAMPLE_FINAL);
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* part = scratch + (size_t)row * chunks * 4;
    // the first maximum over the chunks
    float best = -CUDART_INF_F;
    int arg = 0x7fffffff;
    for (int c = tid; c < chunks; c += SAMPLE_THREADS) argmax_merge(best, arg, part[c * 4], __float_as_int(part[c * 4 + 1]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_merge(best, arg, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, arg, o));
    if (lane == 0) { s_v[warp] = best; s_i[warp] = arg; }
    __syncthreads();
    if (tid == 0) {
        for (int k = 1; k < SAMPLE_THREADS / 32; k++) argmax_merge(best, arg, s_v[k], s_i[k]);
        s_max = best; s_arg = arg;
    }
    __syncthreads();
    const float temp = temperature[row];
    if (!(temp > 0.f)) {
        if (tid == 0) tokens[row] = s_arg;
        return;
    }
    const float inv = 1.0f / temp, top = s_max * inv;
    if (tid == 0) {
        // chunks in their order: total, then the chunk whose span of the running sum holds the point
        float total = 0.f;
        for (int c = 0; c < chunks; c++) total += part[c * 4 + 2] * expf(part[c * 4] * inv - top);
        const float point = uniform[row] * total;
        float run = 0.f;
        int pick = -1;
        float before = 0.f;
        for (int c = 0; c < chunks; c++) {
            const float w = part[c * 4 + 2] * expf(part[c * 4] * inv - top);
            if (run + w >= point && w > 0.f) { pick = c; before = run; break; }
            run += w;
        }
        s_chunk = pick; s_before = before; s_point = point; s_owner = 0x7fffffff;
    }
    __syncthreads();
    if (s_chunk < 0) {  // rounding left the point past every sum: the most likely token
        if (tid == 0) tokens[row] = s_arg;
        return;
    }
    const float* l = logits + (size_t)row * row_stride;
    const int c0 = s_chunk * SAMPLE_CHUNK + tid * SAMPLE_PER_THREAD;   // ids upward: each thread a contiguous run
    const int c1 = min(vocab, c0 + SAMPLE_PER_THREAD);
    float sum = 0.f;
    for (int i = c0; i < c1; i++) sum += expf(l[i] * inv - top);
    float x = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) s_v[warp] = x;
    __syncthreads();
    float offset = s_before;
    for (int k = 0; k < warp; k++) offset += s_v[k];
    const float incl = x + offset;
    s_scan[tid] = incl;
    __syncthreads();
    const float point = s_point;
    if (incl >= point && c1 > c0) atomicMin(&s_owner, tid);
    __syncthreads();
    const int owner = s_owner;
    if (owner == 0x7fffffff) {
        // the chunk's own sums fell short of what its partial promised: its last token
        if (tid == 0) tokens[row] = min(vocab, (s_chunk + 1) * SAMPLE_CHUNK) - 1;
        return;
    }
    if (tid == owner) {
        float run = tid > 0 ? s_scan[tid - 1] : s_before;
        int pick = c1 - 1;
        for (int i = c0; i < c1; i++) {
            run += expf(l[i] * inv - top);
            if (run >= point) { pick = i; break; }
        }
        tokens[row] = pick;
    }
}

// Floats of scratch memory pllm_sample needs for n_rows rows of `vocab` logits.
PLLM_EXPORT long long pllm_sample_scratch_floats(int n_rows, int vocab) {
    const long long chunks = (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    return (long long)n_rows * chunks * 4;
}

PLLM_EXPORT int pllm_sample(const float* logits, int n_rows, int vocab, long long row_stride,
                            const float* temperature, const float* uniform, int* tokens, float* scratch,
                            cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (vocab <= 0) return PLLM_ERR_SIZE;
    const int chunks = (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    launch_chained(sample_partial_kernel, dim3(chunks, n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, vocab,
                   row_stride, temperature, scratch);
    launch_chained(sample_final_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, vocab, row_stride,
                   chunks, temperature, uniform, (const float*)scratch, tokens);
    return launch_status();
}

// ---- sampling without any allocation (declared in sampling_static.h) ------------------------
// This entry point has no counterpart in the reference.  It is for callers that may not
// allocate device memory at all when they ask for a token: code running inside a
// section where cudaMalloc is forbidden or would stall every stream (a real-time
// control loop that holds the device, a plugin loaded into a host process that gave it
// a fixed memory budget at start-up and hands it no allocator), or code that must not
// touch torch's allocator from its thread.  pllm_sample needs scratch memory between
// its two launches and leaves it to the caller to provide; here that scratch is a fixed
// array in the library's own device image, so the call needs nothing but its inputs
// and outputs.
//
// The price: the array is there on every GPU that loads this library, from load to exit,
// whether or not this entry point is ever called (PLLM_STATIC_SAMPLE_FLOATS * 4 bytes =
// 256 KiB), and it bounds what one call may ask for: at most PLLM_STATIC_SAMPLE_MAX_ROWS
// rows of at most PLLM_STATIC_SAMPLE_MAX_VOCAB logits.  Larger requests are refused
// with PLLM_ERR_LIMIT and nothing is launched.
//
// All calls share the one array.  Every entry a call reads it has written itself
// earlier in the same call, so nothing has to be cleared between calls and what an
// earlier call left behind is never seen; but two calls whose kernels overlap on the GPU
// (different streams, no ordering between them) write the same entries and race.
// Keep calls of this entry point ordered on one stream, or order them with events.
//
// The first call on a device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and keeps it; make that first call
// outside any stream capture.  Nothing here calls cudaMalloc, cudaFree or any
// allocating routine of a library.
#include "sampling_static.h"

static __device__ __align__(256) float g_static_sample_scratch[PLLM_STATIC_SAMPLE_FLOATS];

// In host code the array's name stands for a host-side shadow, not for device memory;
// the device address is asked for once per device and kept here.
#define PLLM_MAX_DEVICES 64
static float* g_static_sample_ptr[PLLM_MAX_DEVICES];

PLLM_EXPORT int pllm_sample_static(const float* logits, int n_rows, int vocab, long long row_stride,
                                   const float* temperature, const float* uniform, int* tokens, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (vocab <= 0) return PLLM_ERR_SIZE;
    if (n_rows > PLLM_STATIC_SAMPLE_MAX_ROWS || vocab > PLLM_STATIC_SAMPLE_MAX_VOCAB) return PLLM_ERR_LIMIT;
    const int chunks = (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK;
    if ((long long)n_rows * chunks * 4 > PLLM_STATIC_SAMPLE_FLOATS) return PLLM_ERR_LIMIT;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= PLLM_MAX_DEVICES) return PLLM_ERR_LIMIT;
    float* scratch = g_static_sample_ptr[device];
    if (scratch == nullptr) {
        e = cudaGetSymbolAddress((void**)&scratch, g_static_sample_scratch);
        if (e != cudaSuccess) return (int)e;
        g_static_sample_ptr[device] = scratch;   // the same value whoever stores it first
    }
    launch_chained(sample_partial_kernel, dim3(chunks, n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, vocab,
                   row_stride, temperature, scratch);
    launch_chained(sample_final_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, stream, logits, vocab, row_stride,
                   chunks, temperature, uniform, (const float*)scratch, tokens);
    return launch_status();
}

PLLM_TRACE_EXPORT(sampling)

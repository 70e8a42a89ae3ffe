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
// One CTA per row.  Sums are formed in a fixed order (each thread over its own
// contiguous range, then a scan over threads), so a draw does not depend on
// timing.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__global__ void sample_kernel(const float* __restrict__ logits, int vocab, long long row_stride,
                              const float* __restrict__ temperature,  // [n]; <= 0: greedy
                              const float* __restrict__ uniform,      // [n] in [0, 1)
                              int* __restrict__ tokens) {
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ float s_scan[SAMPLE_THREADS];
    __shared__ float s_max;
    __shared__ int s_arg, s_owner;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* l = logits + (size_t)row * row_stride;
    const int per = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int c0 = min(vocab, tid * per), c1 = min(vocab, c0 + per);

    // first maximum: larger value wins, equal values keep the smaller id
    float best = -CUDART_INF_F;
    int arg = 0x7fffffff;
    for (int i = c0; i < c1; i++) {
        const float v = l[i];
        if (arg == 0x7fffffff || v > best) { best = v; arg = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
    }
    if (lane == 0) { s_val[warp] = best; s_idx[warp] = arg; }
    __syncthreads();
    if (warp == 0) {
        best = s_val[lane]; arg = s_idx[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ov > best || (ov == best && oi < arg)) { best = ov; arg = oi; }
        }
        if (lane == 0) { s_max = best; s_arg = arg; s_owner = 0x7fffffff; }
    }
    __syncthreads();
    const float temp = temperature[row];
    if (!(temp > 0.f)) {
        if (tid == 0) tokens[row] = s_arg;
        return;
    }
    const float inv = 1.0f / temp;
    const float top = s_max * inv;
    float sum = 0.f;
    for (int i = c0; i < c1; i++) sum += expf(l[i] * inv - top);
    // inclusive scan over threads, in thread order
    float x = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) s_val[warp] = x;
    __syncthreads();
    if (warp == 0) {
        float w = s_val[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        s_val[lane] = w;
    }
    __syncthreads();
    const float incl = x + (warp > 0 ? s_val[warp - 1] : 0.f);
    const float total = s_val[31];
    s_scan[tid] = incl;
    __syncthreads();
    const float point = uniform[row] * total;
    // the first thread whose inclusive sum reaches the point owns the draw
    const float before = tid > 0 ? s_scan[tid - 1] : 0.f;
    if (incl >= point && c1 > c0) atomicMin(&s_owner, tid);
    __syncthreads();
    const int owner = s_owner;
    if (owner == 0x7fffffff) {  // rounding left the point past every sum: take the most likely token
        if (tid == 0) tokens[row] = s_arg;
        return;
    }
    if (tid == owner) {
        float run = before;
        int pick = c1 - 1;
        for (int i = c0; i < c1; i++) {
            run += expf(l[i] * inv - top);
            if (run >= point) { pick = i; break; }
        }
        tokens[row] = pick;
    }
}

PLLM_EXPORT int pllm_sample(const float* logits, int n_rows, int vocab, long long row_stride,
                            const float* temperature, const float* uniform, int* tokens, cudaStream_t stream) {
    if (n_rows <= 0) return PLLM_OK;
    if (vocab <= 0) return PLLM_ERR_SIZE;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, stream>>>(logits, vocab, row_stride, temperature, uniform, tokens);
    return launch_status();
}

// What the tcgen05 kernels share: barriers with bounded waits, TMA tile loads, shared-memory and
// instruction descriptors, tcgen05.mma / commit / ld / st, and the host's tensor maps.
//
// Descriptor layouts are those of the PTX ISA's tcgen05 chapter (as CUTLASS's
// cute/arch/mma_sm100_desc.hpp spells them out):
//   shared-memory descriptor: bits 0-13 start address >> 4, 16-29 leading byte offset >> 4,
//     32-45 stride byte offset >> 4, 46-47 version (1), 61-63 layout (2: 128-byte swizzle);
//   instruction descriptor (kind::f16): bits 4-5 accumulator format (1: float), 7-9 A format,
//     10-12 B format (1: bfloat16), 15 A major, 16 B major (0: K, 1: MN), 17-22 N >> 3, 24-28 M >> 4.
// A tile stored with the 128-byte swizzle has rows of 128 bytes in groups of 8 (1024 bytes) whose
// 16-byte chunk c of row r sits at chunk c ^ (r & 7); the tile starts on a 1024-byte boundary.
//   K-major operand (rows = M or N, 64 elements of K a row): stride byte offset 1024; 16 values of
//     k further along = start address + 32 bytes.
//   MN-major operand (rows = K, 64 elements of M or N a row): stride byte offset 1024 between groups
//     of 8 rows of K, leading byte offset = distance to the next 64 elements of M or N.
#pragma once

#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"

namespace tc {

constexpr int SPIN_LIMIT = 1 << 22;

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
// or when another thread has given up.  Returns false then.  (Polling with test_wait, which never
// suspends the thread, measured no faster in the tcgen05 attention.)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int spin = 0; spin < SPIN_LIMIT; spin++) {
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
// (stride_bytes: from one group of 8 rows to the next, 1024 when the groups lie back to back)
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t leading_bytes = 16, uint32_t stride_bytes = 1024) {
    return (uint64_t)((addr >> 4) & 0x3fff) | ((uint64_t)((leading_bytes >> 4) & 0x3fff) << 16) |
           ((uint64_t)((stride_bytes >> 4) & 0x3fff) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: float accumulator, bfloat16 A and B, both K-major, M x N.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, int b_mn_major = 0) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// The same with the A operand in tensor memory: rows are lanes, two 16-bit values of k to a 32-bit column
// (16 values of k = 8 columns), k ascending from the low half.
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n}\n"
                 ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
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

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, int w, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t addr, const uint32_t (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
                 ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// ---- host: tensor maps (bfloat16), kept by what they describe -----------------------------------

struct MapKey {
    const void* ptr; int rank; long long dims[4]; long long strides[3]; int box[4]; int swizzle;
    bool operator<(const MapKey& o) const {
        return std::tie(ptr, rank, dims[0], dims[1], dims[2], dims[3], strides[0], strides[1], strides[2], box[0], box[1], box[2], box[3], swizzle) <
               std::tie(o.ptr, o.rank, o.dims[0], o.dims[1], o.dims[2], o.dims[3], o.strides[0], o.strides[1], o.strides[2], o.box[0], o.box[1],
                        o.box[2], o.box[3], o.swizzle);
    }
};

// dims: elements, innermost first (rank 2 to 4); strides: bytes of dims 1.. ; box: elements.  swizzle128: the
// hardware stores the box with the 128-byte swizzle (the box's innermost extent is then 64 elements).
inline int tensor_map(const void* ptr, int rank, const long long* dims, const long long* strides, const int* box,
                      bool swizzle128, CUtensorMap* out) {
    static std::map<MapKey, CUtensorMap> maps;
    static std::mutex lock;
    std::lock_guard<std::mutex> hold(lock);
    if (rank < 2 || rank > 4) return -1;
    MapKey key{ptr, rank, {1, 1, 1, 1}, {0, 0, 0}, {1, 1, 1, 1}, swizzle128 ? 1 : 0};
    for (int i = 0; i < rank; i++) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    for (int i = 0; i + 1 < rank; i++) key.strides[i] = strides[i];
    auto it = maps.find(key);
    if (it != maps.end()) { *out = it->second; return 0; }
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
    cuuint64_t d[4], st[3];
    cuuint32_t b[4], e[4] = {1, 1, 1, 1};
    for (int i = 0; i < 4; i++) { d[i] = (cuuint64_t)key.dims[i]; b[i] = (cuuint32_t)key.box[i]; }
    for (int i = 0; i < 3; i++) st[i] = (cuuint64_t)key.strides[i];
    const CUresult r = encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), d, st, b, e,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return (int)r;
    if (maps.size() > 4096) maps.clear();     // activations come and go; weights come back
    maps[key] = *out;
    return 0;
}

}  // namespace tc

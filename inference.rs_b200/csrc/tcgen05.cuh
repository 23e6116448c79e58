// Wrappers around the sm_100a instructions the tensor-core kernels share: tiled TMA loads, tensor-memory allocation,
// tcgen05.mma / commit / ld, shared-memory operand descriptors, and the host lookup of cuTensorMapEncodeTiled.
#pragma once
#include <mutex>
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace b200q {

// ---- tcgen05 / TMA wrappers ------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* dst_smem, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], 16-bit inputs, f32 accumulate
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread (thread = lane of this warp's TMEM quarter)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, "
        "%18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
// Descriptor fields: start address >> 4 (14 bits), leading byte offset (unused for swizzled K-major, 1),
// stride byte offset 1024 >> 4 at bit 32, descriptor version 1 at bit 46, layout type SWIZZLE_128B (2) at bit 61.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t smem_addr) {
    return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: f32 accumulator (1 at bit 4), A / B format at bits 7 / 10 (0 = f16, 1 = bf16),
// both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_f16(int fmt, int m, int n) {
    return (1u << 4) | ((uint32_t)fmt << 7) | ((uint32_t)fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// 16-byte chunk j of row r of a K-major 128-byte-swizzled operand tile (rows of 128 bytes): its swizzled position.
__device__ __forceinline__ uint32_t b_chunk_addr(uint32_t stage_addr, int r, int j) {
    return stage_addr + (uint32_t)(r >> 3) * 1024u + (uint32_t)(r & 7) * 128u + (uint32_t)((j ^ (r & 7)) << 4);
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// kind::i8: 8-bit integer inputs (32 per row and instruction), s32 accumulate. `accumulate` as above.
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor, kind::i8: s32 accumulator (2 at bit 4), A / B format at bits 7 / 10 (0 = unsigned, 1 = signed
// 8-bit), both K-major, N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_i8(int a_signed, int b_signed, int m, int n) {
    return (2u << 4) | ((uint32_t)a_signed << 7) | ((uint32_t)b_signed << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
// 32 lanes x 4 consecutive 32-bit columns -> 4 registers per thread; the caller waits with tmem_ld_wait()
__device__ __forceinline__ void tmem_ld_32x4_nowait(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        else
            cudaGetLastError();
    }
    return fn;
}

// cuTensorMapEncodeTiled for a 2-D map, remembered by its arguments: a decoder calls the same matrices with the same
// shapes every step, and the encoding (a driver call of a microsecond or two on the host) depends on nothing else - a
// map only describes an address range. A small direct-mapped table per translation unit, guarded by a mutex.
struct TensorMapKey {
    const void* ptr;
    unsigned long long dim0, dim1, stride0;
    unsigned int box0, box1;
    int dtype, swizzle, l2;
    bool operator==(const TensorMapKey& o) const {
        return ptr == o.ptr && dim0 == o.dim0 && dim1 == o.dim1 && stride0 == o.stride0 && box0 == o.box0 && box1 == o.box1 &&
               dtype == o.dtype && swizzle == o.swizzle && l2 == o.l2;
    }
};
static inline CUresult encode_tiled_2d_cached(CUtensorMap* out, CUtensorMapDataType dt, const void* ptr, const cuuint64_t (&dims)[2],
                                             cuuint64_t stride0, const cuuint32_t (&box)[2], CUtensorMapSwizzle swizzle,
                                             CUtensorMapL2promotion l2) {
    constexpr int SLOTS = 256;
    struct Slot { TensorMapKey key; CUtensorMap map; bool used; };
    static Slot table[SLOTS];
    static std::mutex mu;
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return CUDA_ERROR_NOT_SUPPORTED;
    const TensorMapKey key{ptr, dims[0], dims[1], stride0, box[0], box[1], (int)dt, (int)swizzle, (int)l2};
    unsigned long long h = reinterpret_cast<unsigned long long>(ptr) >> 4;
    h = (h ^ (dims[1] * 0x9E3779B97F4A7C15ull) ^ (dims[0] << 7) ^ box[1]) * 0xD6E8FEB86659FD93ull;
    Slot& slot = table[(h >> 40) % SLOTS];
    {
        std::lock_guard<std::mutex> lock(mu);
        if (slot.used && slot.key == key) {
            *out = slot.map;
            return CUDA_SUCCESS;
        }
    }
    const cuuint64_t strides[1] = {stride0};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(out, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, l2,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        std::lock_guard<std::mutex> lock(mu);
        slot.key = key;
        slot.map = *out;
        slot.used = true;
    }
    return r;
}

}  // namespace b200q

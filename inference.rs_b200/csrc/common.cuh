// Shared definitions for the sm_100a GGUF quantized-matmul kernels: GGUF block layouts (unchanged from
// the file format), PTX wrappers for mbarrier / bulk-copy (TMA) staging, bounded waits and the device
// status word.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {

// ---------------------------------------------------------------------------------------------
// GGUF block layouts (little endian, no padding). Same bytes as the reference reads:
// crates/inference-tensor/src/quantized/k_quants.rs:150-227.
// ---------------------------------------------------------------------------------------------
constexpr int QK_K = 256;
constexpr int QK8 = 32;

constexpr int Q8_0_BYTES = 34;   // f16 d; i8 qs[32]
constexpr int Q8_1_BYTES = 36;   // f16 d; f16 s; i8 qs[32]
constexpr int Q4_K_BYTES = 144;  // f16 d; f16 dmin; u8 scales[12]; u8 qs[128]
constexpr int Q6_K_BYTES = 210;  // u8 ql[128]; u8 qh[64]; i8 scales[16]; f16 d
constexpr int MMQ_BLOCK_BYTES = 144;  // prefill activation block: 16 B of scales + 128 i8

// GGUF type ids (crates/inference-tensor/src/quantized/mod.rs:582-624)
enum GgmlType : int { TYPE_Q8_0 = 8, TYPE_Q4_K = 12, TYPE_Q6_K = 14 };
// activation / output element types of the launchers
enum ElemType : int { ELEM_F32 = 0, ELEM_F16 = 1, ELEM_BF16 = 2 };

__host__ __device__ constexpr int type_block_elems(int t) { return t == TYPE_Q8_0 ? 32 : 256; }
__host__ __device__ constexpr int type_block_bytes(int t) {
    return t == TYPE_Q8_0 ? Q8_0_BYTES : (t == TYPE_Q4_K ? Q4_K_BYTES : (t == TYPE_Q6_K ? Q6_K_BYTES : 0));
}

// ---------------------------------------------------------------------------------------------
// Device status word. A kernel that gives up on a wait records why here instead of trapping; the host
// reads it with b200q_device_status(). 0 = ok.
// ---------------------------------------------------------------------------------------------
enum DeviceStatus : unsigned int {
    STATUS_OK = 0,
    STATUS_WAIT_FULL_TIMEOUT = 1,   // a consumer gave up waiting for a staged tile
    STATUS_WAIT_EMPTY_TIMEOUT = 2,  // the producer gave up waiting for a free stage
    STATUS_WAIT_MMA_TIMEOUT = 3,    // the epilogue gave up waiting for the tensor core
    STATUS_WAIT_DRAIN_TIMEOUT = 4,  // copies still in flight at exit did not land in time
    STATUS_WAIT_PEER_TIMEOUT = 5,   // a peer rank's flag did not arrive in time
    STATUS_BAD_ROW_ID = 6,          // a row gather was given an id outside the table (that output row is zero)
};

// The word lives in one translation unit (runtime.cu); kernels receive its device address as a parameter
// (status_ptr() on the host). Layout: [0] first failure code, [1] block, [2] detail, [3] number of failures.
__device__ __forceinline__ void record_failure(unsigned int* status, unsigned int code, unsigned int detail) {
    if (status == nullptr) return;
    if (atomicCAS(&status[0], 0u, code) == 0u) {
        status[1] = blockIdx.x;
        status[2] = detail;
    }
    atomicAdd(&status[3], 1u);
}

// ---------------------------------------------------------------------------------------------
// Small numeric helpers
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
    return __half2float(__ushort_as_half((unsigned short)(bits16 & 0xffffu)));
}

// a (4 unsigned bytes) . b (4 signed bytes) + c
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
// a (4 signed bytes) . b (4 signed bytes) + c
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
    return v;
}
__device__ __forceinline__ int warp_sum_int(int v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// ---------------------------------------------------------------------------------------------
// Shared-memory barriers and bulk (TMA) copies
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Every wait in these kernels is bounded: about a second of polling, then the caller records a failure
// and leaves. Returns false on timeout.
constexpr uint32_t WAIT_SPINS = 1u << 22;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < WAIT_SPINS; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    return false;
}

// Two barriers at once (see mbar_wait3_bounded).
__device__ __forceinline__ bool mbar_wait2_bounded(uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1) {
    bool d0 = false, d1 = false;
    for (uint32_t i = 0; i < WAIT_SPINS; ++i) {
        const bool t0 = d0 || mbar_try_wait(b0, p0);
        const bool t1 = d1 || mbar_try_wait(b1, p1);
        d0 = t0;
        d1 = t1;
        if (d0 && d1) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    return false;
}

// Three barriers at once: the polls are issued back to back so that their shared-memory round trips overlap (a poll
// queues behind whatever loads and stores the CTA's other warps have in flight, which can be hundreds of cycles).
__device__ __forceinline__ bool mbar_wait3_bounded(uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1, uint64_t* b2, uint32_t p2) {
    bool d0 = false, d1 = false, d2 = false;
    for (uint32_t i = 0; i < WAIT_SPINS; ++i) {
        const bool t0 = d0 || mbar_try_wait(b0, p0);
        const bool t1 = d1 || mbar_try_wait(b1, p1);
        const bool t2 = d2 || mbar_try_wait(b2, p2);
        d0 = t0;
        d1 = t1;
        d2 = t2;
        if (d0 && d1 && d2) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    return false;
}

// 1-D bulk copy global -> shared through the TMA unit; completion counted in bytes on `bar`.
// dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// generic-proxy writes to shared memory made visible to the async proxy (TMA / tensor core reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// programmatic dependent launch: wait for the previous grid in the stream (no-op when not launched that way)
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Explicit shared-space loads on 32-bit shared addresses: keeps the compiler from falling back to generic loads
// (64-bit address arithmetic, long-scoreboard latency) for pointers it cannot prove to be shared.
__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint32_t v;
    asm volatile("{ .reg .u16 t; ld.shared.u16 t, [%1]; cvt.u32.u16 %0, t; }" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ float lds_f32(uint32_t a) { return __uint_as_float(lds32(a)); }

// `NW` 32-bit words starting `O` bytes (even, compile time) into the 16-byte-aligned words c[]
template <int O, int NW, int NC>
__device__ __forceinline__ void extract_words(const uint32_t (&c)[NC], uint32_t (&out)[NW]) {
    constexpr int wo = O >> 2;
#pragma unroll
    for (int i = 0; i < NW; ++i) {
        if constexpr ((O & 2) == 0) {
            out[i] = c[wo + i];
        } else if constexpr (wo + NW < NC) {
            out[i] = __funnelshift_r(c[wo + i], c[wo + i + 1], 16);
        } else {
            // the last word's upper half would come from beyond c[]: the callers only use its lower half
            out[i] = (wo + i + 1 < NC) ? __funnelshift_r(c[wo + i], c[(wo + i + 1 < NC) ? wo + i + 1 : NC - 1], 16) : (c[wo + i] >> 16);
        }
    }
}
template <int NCHUNK>
__device__ __forceinline__ void lds_chunks(uint32_t addr, uint32_t (&c)[4 * NCHUNK]) {
#pragma unroll
    for (int i = 0; i < NCHUNK; ++i) {
        const uint4 v = lds128(addr + 16 * i);
        c[4 * i] = v.x; c[4 * i + 1] = v.y; c[4 * i + 2] = v.z; c[4 * i + 3] = v.w;
    }
}


// int -> float without the conversion unit: exact for |v| < 2^22 (adds v ulps to 1.5 * 2^23, then subtracts it)
__device__ __forceinline__ float int_to_float_small(int v) { return __int_as_float(0x4B400000 + v) - 12582912.0f; }

// An aligned 32-bit word read at a 2-byte-aligned address: two aligned loads and a funnel shift.
__device__ __forceinline__ uint32_t funnel16(uint32_t lo, uint32_t hi, uint32_t shift_bits) {
    return __funnelshift_r(lo, hi, shift_bits);
}

}  // namespace b200q

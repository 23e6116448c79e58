// Device side of the one-shot sum all-reduce over peer-mapped buffers (protocol and buffer layout: peer_allreduce.cu),
// shared by the stand-alone kernel and by the GEMV whose last CTA runs it on the matmul's own output.
#pragma once
#include "common.cuh"

namespace b200q {

constexpr int PAR_MAX_WORLD = 8;
constexpr int PAR_MAX_BLOCKS = 7;
constexpr int PAR_HEADER_BYTES = 1024;
constexpr int PAR_EPOCH_OFFSET = 768;
constexpr int PAR_THREADS = 512;

constexpr int PAR_COUNTER_OFFSET = 832;  // arrival counter of the CTAs of a fused matmul + all-reduce launch
constexpr int PAR_FUSED_BLOCK = 7;       // flag / epoch slot of the fused path (stand-alone calls use blocks 0..6)

// The ranks' exchange buffers as mapped in this process; world <= 1 means "no exchange".
struct PeerExchange {
    uint8_t* bufs[PAR_MAX_WORLD];  // bufs[rank] is the local one
    long long capacity;            // bytes of one staging half
    int rank, world;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// peer data is read past the L1 cache: the same addresses carry new values every second call
__device__ __forceinline__ uint4 ld_volatile_16(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

template <typename T> struct Vec16;  // 16 bytes of T <-> floats
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void add(const uint4& u, float (&a)[8]) {
        a[0] += __uint_as_float(u.x); a[1] += __uint_as_float(u.y); a[2] += __uint_as_float(u.z); a[3] += __uint_as_float(u.w);
    }
    static __device__ __forceinline__ uint4 pack(const float (&a)[8]) {
        return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3]));
    }
};
template <> struct Vec16<__half> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void add(const uint4& u, float (&a)[8]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            a[2 * i] += f.x;
            a[2 * i + 1] += f.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&a)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __half2 h = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void add(const uint4& u, float (&a)[8]) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
            a[2 * i] += f.x;
            a[2 * i + 1] += f.y;
        }
    }
    static __device__ __forceinline__ uint4 pack(const float (&a)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// One slice [u0, u1) (16-byte units) of the vector, by `nthreads` threads of one CTA (tid < nthreads; all of them must
// call). `staging` = byte offset of the two staging halves in every rank's buffer, `slot` = which flag / epoch slot.
// NAMED: the threads are a subset of the CTA that meets on named barrier 1; else the whole CTA (__syncthreads).
// `scratch` = two words of shared memory. Returns false (on all threads) if a peer did not arrive in time.
template <typename T, bool NAMED>
__device__ __forceinline__ bool peer_allreduce_slice(const PeerExchange& px, size_t staging, int slot, const void* in, void* out,
                                                     long long u0, long long u1, int tid, int nthreads, unsigned int* status,
                                                     volatile unsigned int* scratch) {
    using V = Vec16<T>;
    uint8_t* mine = px.bufs[px.rank];
    if (tid == 0) {
        unsigned int* epoch = reinterpret_cast<unsigned int*>(mine + PAR_EPOCH_OFFSET) + slot;
        const unsigned int e1 = *epoch + 1u;
        *epoch = e1;
        scratch[0] = e1;
        scratch[1] = 1u;
    }
    if (NAMED) named_bar_sync(1, nthreads); else __syncthreads();
    const unsigned int e = scratch[0];
    const size_t half_off = staging + (size_t)(e & 1u) * (size_t)px.capacity;

    // 1. this rank's slice into its staging half (read past L1: other CTAs may have produced it)
    {
        const uint4* src = reinterpret_cast<const uint4*>(in);
        uint4* dst = reinterpret_cast<uint4*>(mine + half_off);
        for (long long u = u0 + tid; u < u1; u += nthreads) dst[u] = __ldcg(src + u);
    }
    __threadfence_system();
    if (NAMED) named_bar_sync(1, nthreads); else __syncthreads();

    // 2. tell every rank, then wait for every rank
    if (tid < px.world) {
        st_release_sys(reinterpret_cast<unsigned int*>(px.bufs[tid]) + slot * 16 + px.rank, e);
        const unsigned int* flag = reinterpret_cast<const unsigned int*>(mine) + slot * 16 + tid;
        bool ok = false;
        for (unsigned int spin = 0; spin < WAIT_SPINS; ++spin) {
            if ((int)(ld_acquire_sys(flag) - e) >= 0) {
                ok = true;
                break;
            }
            if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
        }
        if (!ok) {
            scratch[1] = 0u;
            record_failure(status, STATUS_WAIT_PEER_TIMEOUT, (unsigned int)(slot * 16 + tid));
        }
    }
    if (NAMED) named_bar_sync(1, nthreads); else __syncthreads();
    if (scratch[1] == 0u) return false;

    // 3. the same sum in the same order on every rank
    uint4* o = reinterpret_cast<uint4*>(out);
    for (long long u = u0 + tid; u < u1; u += nthreads) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < px.world; ++r) V::add(ld_volatile_16(px.bufs[r] + half_off + (size_t)u * 16), acc);
        o[u] = V::pack(acc);
    }
    return true;
}

}  // namespace b200q

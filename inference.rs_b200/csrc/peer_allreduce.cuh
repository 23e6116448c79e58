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
constexpr int PAR_FUSED_BLOCK = 7;       // flag / epoch slot of the fused path (stand-alone calls use slots 0..6)

// The ranks' exchange buffers as mapped in this process; world <= 1 means "no exchange".
struct PeerExchange {
    uint8_t* bufs[PAR_MAX_WORLD];  // bufs[rank] is the local one
    long long capacity;            // largest vector in bytes
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

// ---- buffer layout (every rank's buffer is the same; `capacity` = largest vector in bytes, a multiple of 16) ----
//   [0, 512)      arrive[slot 0..7][source rank 0..15]  u32, written by the peers
//   768           epoch[slot 0..7]                       u32, local
//   832           arrival counter of the CTAs of a fused matmul + all-reduce launch
//   [1024, ...)   inboxes: for stand-alone slot i < 7, half h, source rank r: slot_cap bytes at
//                 1024 + ((i * 2 + h) * 8 + r) * slot_cap, slot_cap = ceil16(capacity / 7): slot i always carries bytes
//                 [i * slot_cap, (i + 1) * slot_cap) of a vector, whatever the vector's length, so a slot's inboxes
//                 only ever meet that slot's own earlier calls;
//                 then the fused launches' inboxes (slot 7): capacity bytes at fused_base + (h * 8 + r) * capacity.
__host__ __device__ inline long long par_slot_cap(long long capacity) { return ((capacity + PAR_MAX_BLOCKS - 1) / PAR_MAX_BLOCKS + 15) & ~15LL; }
__host__ __device__ inline long long par_inbox_offset(long long capacity, int slot, unsigned int half, int src) {
    return PAR_HEADER_BYTES + (((long long)slot * 2 + half) * PAR_MAX_WORLD + src) * par_slot_cap(capacity);
}
__host__ __device__ inline long long par_fused_base(long long capacity) {
    return PAR_HEADER_BYTES + (long long)PAR_MAX_BLOCKS * 2 * PAR_MAX_WORLD * par_slot_cap(capacity);
}
__host__ __device__ inline long long par_fused_inbox_offset(long long capacity, unsigned int half, int src) {
    return par_fused_base(capacity) + ((long long)half * PAR_MAX_WORLD + src) * capacity;
}
__host__ __device__ inline long long par_buffer_bytes(long long capacity) { return par_fused_base(capacity) + 2LL * PAR_MAX_WORLD * capacity; }

__device__ __forceinline__ void st_global_16(void* p, const uint4& v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Second half of an exchange, by `nthreads` threads of one CTA (tid < nthreads; all of them must call): every rank's
// contribution to units [0, nunits) of this slot has been pushed into the peers' inboxes (at `inbox0` + source rank *
// `inbox_stride` of the epoch's half) and fenced at system scope by the threads that wrote it. Raises this rank's flag
// in every peer, waits - bounded - for every peer's flag, then adds the `world` inboxes of the LOCAL buffer in rank
// order in f32 and stores units of `out`. NAMED: the threads are a subset of the CTA that meets on named barrier 1.
// `scratch` = one word of shared memory. Returns false (on all threads) if a peer did not arrive in time.
template <typename T, bool NAMED>
__device__ __forceinline__ bool peer_signal_wait_reduce(const PeerExchange& px, int slot, unsigned int e, long long inbox0,
                                                        long long inbox_stride, void* out, long long nunits, int tid, int nthreads,
                                                        unsigned int* status, volatile unsigned int* scratch) {
    using V = Vec16<T>;
    uint8_t* mine = px.bufs[px.rank];
    if (tid == 0) scratch[0] = 1u;
    if (NAMED) named_bar_sync(1, nthreads); else __syncthreads();
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
            scratch[0] = 0u;
            record_failure(status, STATUS_WAIT_PEER_TIMEOUT, (unsigned int)(slot * 16 + tid));
        }
    }
    if (NAMED) named_bar_sync(1, nthreads); else __syncthreads();
    if (scratch[0] == 0u) return false;
    // the same sum in the same order on every rank, from local memory
    uint4* o = reinterpret_cast<uint4*>(out);
    for (long long u = tid; u < nunits; u += nthreads) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < px.world; ++r) V::add(ld_volatile_16(mine + inbox0 + r * inbox_stride + (size_t)u * 16), acc);
        o[u] = V::pack(acc);
    }
    return true;
}

}  // namespace b200q

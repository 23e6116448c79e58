// Device side of the one-shot sum all-reduce over peer-mapped buffers (protocol and buffer layout: peer_allreduce.cu),
// shared by the stand-alone kernel and by the GEMVs whose CTAs run it on their own rows of the matmul's output.
#pragma once
#include "common.cuh"

namespace b200q {

constexpr int PAR_MAX_WORLD = 8;
constexpr int PAR_HEADER_BYTES = 1024;
constexpr int PAR_THREADS = 256;
// header words (u32, read and written by the owning rank only)
constexpr int PAR_EPOCH_ALONE = 0;    // number of the last finished stand-alone call
constexpr int PAR_COUNT_ALONE = 1;    // finished blocks of the running stand-alone call
constexpr int PAR_EPOCH_FUSED = 2;    // number of the last finished matmul + all-reduce launch
constexpr int PAR_COUNT_FUSED = 3;    // finished CTAs of the running one
constexpr int PAR_PATH_ALONE = 0, PAR_PATH_FUSED = 1;

// The ranks' exchange buffers as mapped in this process; world <= 1 means "no exchange".
struct PeerExchange {
    uint8_t* bufs[PAR_MAX_WORLD];  // bufs[rank] is the local one
    long long capacity;            // largest vector in bytes
    int rank, world;
};

// ---- buffer layout (every rank's buffer is the same; `capacity` = largest vector in bytes, a multiple of 16) ----
//   [0, 16)       the four header words above
//   [1024, ...)   inboxes: for path p (stand-alone calls, fused launches), half h, source rank r, 2 * capacity bytes at
//                 1024 + ((p * 2 + h) * 8 + r) * 2 * capacity.
// An inbox holds a vector as 16-byte cells {payload, call number, payload, call number}: every 8 bytes of the vector
// travel with the number of the call they belong to, in ONE store, so a reader that finds both numbers equal to its own
// call's has the data - no flag to raise afterwards, no fence between data and flag, one NVLink crossing in all. (The
// pairing of a payload word with the number next to it is what the exchange relies on, as NCCL's low-latency protocol
// does.) Call numbers start at 1 on a zeroed buffer and skip 0 when they wrap.
__host__ __device__ inline long long par_inbox_offset(long long capacity, int path, unsigned int half, int src) {
    return PAR_HEADER_BYTES + (((long long)path * 2 + half) * PAR_MAX_WORLD + src) * 2 * capacity;
}
__host__ __device__ inline long long par_buffer_bytes(long long capacity) { return PAR_HEADER_BYTES + 4LL * PAR_MAX_WORLD * 2 * capacity; }

__device__ __forceinline__ unsigned int par_next_epoch(unsigned int finished) {
    unsigned int e = finished + 1u;
    return e == 0u ? 2u : e;  // 0 is what a fresh buffer holds; skipping two numbers keeps the halves alternating
}
__device__ __forceinline__ unsigned int* par_header(const PeerExchange& px) { return reinterpret_cast<unsigned int*>(px.bufs[px.rank]); }

// cell `i` of an inbox <- 8 bytes of the vector, stamped with call number e
__device__ __forceinline__ void ll_store(uint8_t* inbox, long long i, uint2 v, unsigned int e) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(inbox + i * 16), "r"(v.x), "r"(e), "r"(v.y), "r"(e) : "memory");
}
// cell `i` of a local inbox, once it carries call number e; false after WAIT_SPINS polls without it
__device__ __forceinline__ bool ll_load(const uint8_t* inbox, long long i, unsigned int e, uint2& v) {
    for (unsigned int spin = 0; spin < WAIT_SPINS; ++spin) {
        uint4 c;
        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(c.x), "=r"(c.y), "=r"(c.z), "=r"(c.w) : "l"(inbox + i * 16) : "memory");
        if (c.y == e && c.w == e) {
            v = make_uint2(c.x, c.z);
            return true;
        }
        if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
    }
    return false;
}

// 8 bytes of T <-> floats
template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static constexpr int N = 2;
    static __device__ __forceinline__ void add(const uint2& u, float (&a)[4]) { a[0] += __uint_as_float(u.x); a[1] += __uint_as_float(u.y); }
    static __device__ __forceinline__ uint2 pack(const float (&a)[4]) { return make_uint2(__float_as_uint(a[0]), __float_as_uint(a[1])); }
};
template <> struct Vec8<__half> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void add(const uint2& u, float (&a)[4]) {
        const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), hi = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        a[0] += lo.x; a[1] += lo.y; a[2] += hi.x; a[3] += hi.y;
    }
    static __device__ __forceinline__ uint2 pack(const float (&a)[4]) {
        const __half2 lo = __floats2half2_rn(a[0], a[1]), hi = __floats2half2_rn(a[2], a[3]);
        return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
};
template <> struct Vec8<__nv_bfloat16> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void add(const uint2& u, float (&a)[4]) {
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        a[0] += lo.x; a[1] += lo.y; a[2] += hi.x; a[3] += hi.y;
    }
    static __device__ __forceinline__ uint2 pack(const float (&a)[4]) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(a[0], a[1]), hi = __floats2bfloat162_rn(a[2], a[3]);
        return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    }
};

// One 8-byte piece of the vector (piece index i): pushes this rank's value into its inbox on EVERY rank (the own buffer
// included), then waits - bounded - for the piece from every rank in the local inboxes and returns their sum, added in
// rank order in f32: every rank computes the same sum in the same order, so all ranks hold identical bits.
// Returns false when a peer's piece did not come in time (STATUS_WAIT_PEER_TIMEOUT is recorded; `sum` is not valid).
template <typename T>
__device__ __forceinline__ void peer_push_piece(const PeerExchange& px, int path, unsigned int e, long long i, uint2 mine) {
    const long long off = par_inbox_offset(px.capacity, path, e & 1u, px.rank);
    for (int r = 0; r < px.world; ++r) ll_store(px.bufs[r] + off, i, mine, e);
}
template <typename T>
__device__ __forceinline__ bool peer_sum_piece(const PeerExchange& px, int path, unsigned int e, long long i, uint2& sum, unsigned int* status) {
    const uint8_t* base = px.bufs[px.rank];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < px.world; ++r) {
        uint2 v;
        if (!ll_load(base + par_inbox_offset(px.capacity, path, e & 1u, r), i, e, v)) {
            record_failure(status, STATUS_WAIT_PEER_TIMEOUT, (unsigned int)r);
            return false;
        }
        Vec8<T>::add(v, acc);
    }
    sum = Vec8<T>::pack(acc);
    return true;
}

// The last block / CTA of a call to finish (local arrival counter) publishes the call number: every block has read the
// previous one by then. Called by one thread per block after the block's pieces are done.
__device__ __forceinline__ void peer_finish_call(const PeerExchange& px, int epoch_word, int count_word, unsigned int e, unsigned int nblocks) {
    unsigned int* hdr = par_header(px);
    const unsigned int before = atomicAdd(hdr + count_word, 1u);
    if (before == nblocks - 1u) {
        hdr[count_word] = 0u;
        *reinterpret_cast<volatile unsigned int*>(hdr + epoch_word) = e;
    }
}

}  // namespace b200q

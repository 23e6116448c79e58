// One-shot sum all-reduce of a small vector over NVLink peer memory: the exchange step after every row-parallel matmul
// of the tensor-parallel decode path (attn_output, ffn_down: [rows, hidden] partial outputs, 16 KB at one row of a
// 70B-class model). Takes the place of the NCCL all-reduce behind the reference's SumAllReduce
// (crates/inference-quant/src/distributed/mod.rs:516-670) where latency, not bandwidth, is the cost: at 8 GPUs a 16 KB
// NCCL all-reduce is a launch of its own of some tens of microseconds, 160 times per token.
//
// Every rank owns one buffer of the same layout, mapped into every other rank's address space (the caller provides the
// mappings; the Python side gets them from torch's symmetric memory):
//   bytes [0, 1024)                flags: arrive[block][source rank] (u32, written by the peers), epoch[block] at 768
//   [1024, 1024 + cap)             staging, epochs with bit 0 clear
//   [1024 + cap, 1024 + 2 cap)     staging, epochs with bit 0 set
// A call on every rank (same sizes everywhere) runs up to eight independent blocks, each on its own slice of the vector:
//   1. e = ++epoch[block]; copy the slice of `in` into the own staging half e & 1; system-scope fence;
//   2. write e into arrive[block][my rank] of every peer (release), then wait until every arrive[block][r] of the own
//      buffer has reached e (acquire): all peers' slices are in place;
//   3. read the slice from every rank's staging half in rank order, add in f32, store to `out`: every rank computes the
//      same sum in the same order, so all ranks hold identical bits.
// The two staging halves make a second barrier unnecessary: a peer rewrites the half of epoch e only in its call e + 2,
// which it enters after its call e + 1 has seen this rank's signal e + 1, sent after this rank finished reading in
// call e. Everything is device-side (no host-provided sequence numbers), so a captured call can be replayed.
// The wait is bounded: a rank that never arrives makes the others record STATUS_WAIT_PEER_TIMEOUT in the device status
// word and return without writing `out`; nothing traps, nothing spins forever.
#include "common.cuh"
#include "runtime.h"

namespace b200q {

constexpr int PAR_MAX_WORLD = 8;
constexpr int PAR_MAX_BLOCKS = 8;
constexpr int PAR_HEADER_BYTES = 1024;
constexpr int PAR_EPOCH_OFFSET = 768;
constexpr int PAR_THREADS = 512;

struct PeerAllReduceParams {
    uint8_t* bufs[PAR_MAX_WORLD];  // every rank's buffer as mapped here; bufs[rank] is the local one
    const void* in;
    void* out;
    long long n;         // elements
    long long capacity;  // bytes of one staging half
    int rank, world;
    unsigned int* status;
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

// `in`, `out` 16-byte aligned, n a multiple of Vec16<T>::N (the host checks)
template <typename T>
__global__ void __launch_bounds__(PAR_THREADS) peer_allreduce_kernel(const PeerAllReduceParams p) {
    using V = Vec16<T>;
    const int blk = blockIdx.x, tid = threadIdx.x;
    const long long units = p.n / V::N;  // 16-byte units
    const long long per_block = (units + gridDim.x - 1) / gridDim.x;
    const long long u0 = blk * per_block, u1 = min(units, u0 + per_block);

    uint8_t* mine = p.bufs[p.rank];
    __shared__ unsigned int s_epoch;
    if (tid == 0) {
        unsigned int* epoch = reinterpret_cast<unsigned int*>(mine + PAR_EPOCH_OFFSET) + blk;
        s_epoch = *epoch + 1u;
        *epoch = s_epoch;
    }
    __syncthreads();
    const unsigned int e = s_epoch;
    const size_t half_off = PAR_HEADER_BYTES + (size_t)(e & 1u) * (size_t)p.capacity;

    // 1. this rank's slice into its staging half
    {
        const uint4* src = reinterpret_cast<const uint4*>(p.in);
        uint4* dst = reinterpret_cast<uint4*>(mine + half_off);
        for (long long u = u0 + tid; u < u1; u += PAR_THREADS) dst[u] = src[u];
    }
    __threadfence_system();
    __syncthreads();

    // 2. tell every rank, then wait for every rank
    bool ok = true;
    if (tid < p.world) {
        st_release_sys(reinterpret_cast<unsigned int*>(p.bufs[tid]) + blk * 16 + p.rank, e);
        const unsigned int* flag = reinterpret_cast<const unsigned int*>(mine) + blk * 16 + tid;
        ok = false;
        for (unsigned int spin = 0; spin < WAIT_SPINS; ++spin) {
            if ((int)(ld_acquire_sys(flag) - e) >= 0) {
                ok = true;
                break;
            }
            if (spin > 64) __nanosleep(spin > 4096 ? 256 : 32);
        }
        if (!ok) record_failure(p.status, STATUS_WAIT_PEER_TIMEOUT, (unsigned int)(blk * 16 + tid));
    }
    if (!__syncthreads_and(ok ? 1 : 0)) return;

    // 3. the same sum in the same order on every rank
    uint4* out = reinterpret_cast<uint4*>(p.out);
    for (long long u = u0 + tid; u < u1; u += PAR_THREADS) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < p.world; ++r) V::add(ld_volatile_16(p.bufs[r] + half_off + (size_t)u * 16), acc);
        out[u] = V::pack(acc);
    }
}

long long peer_allreduce_buffer_bytes(long long capacity) { return PAR_HEADER_BYTES + 2 * capacity; }

int peer_allreduce(const void* const* bufs, int rank, int world, long long capacity, int elem, const void* in, void* out, long long n,
                   cudaStream_t s) {
    if (world < 1 || world > PAR_MAX_WORLD || rank < 0 || rank >= world || capacity <= 0 || capacity % 16 != 0) return B200Q_ERR_INVALID;
    const int esize = elem == ELEM_F32 ? 4 : 2;
    if (n <= 0) return 0;
    if (n * esize > capacity) return B200Q_ERR_TOO_LARGE;
    if ((n * esize) % 16 != 0 || reinterpret_cast<uintptr_t>(in) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0) return B200Q_ERR_UNSUPPORTED;
    PeerAllReduceParams p{};
    for (int r = 0; r < world; ++r) {
        if (bufs[r] == nullptr || reinterpret_cast<uintptr_t>(bufs[r]) % 16 != 0) return B200Q_ERR_INVALID;
        p.bufs[r] = static_cast<uint8_t*>(const_cast<void*>(bufs[r]));
    }
    p.in = in;
    p.out = out;
    p.n = n;
    p.capacity = capacity;
    p.rank = rank;
    p.world = world;
    p.status = status_ptr();
    // one block per 8 KB, at most eight: every rank derives the same count from the same sizes
    long long blocks = (n * esize + 8191) / 8192;
    if (blocks > PAR_MAX_BLOCKS) blocks = PAR_MAX_BLOCKS;
    if (elem == ELEM_F32) peer_allreduce_kernel<float><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_F16) peer_allreduce_kernel<__half><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_BF16) peer_allreduce_kernel<__nv_bfloat16><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else return B200Q_ERR_INVALID;
    return (int)cudaGetLastError();
}

}  // namespace b200q

// One-shot sum all-reduce of a small vector over NVLink peer memory: the exchange step after every row-parallel matmul
// of the tensor-parallel decode path (attn_output, ffn_down: [rows, hidden] partial outputs, 16 KB at one row of a
// 70B-class model). Takes the place of the NCCL all-reduce behind the reference's SumAllReduce
// (crates/inference-quant/src/distributed/mod.rs:516-670) where latency, not bandwidth, is the cost: at 8 GPUs a 16 KB
// NCCL all-reduce is a launch of its own of some tens of microseconds, 160 times per token.
//
// Every rank owns one buffer of the same layout (peer_allreduce.cuh), mapped into every other rank's address space (the
// caller provides the mappings; the Python side gets them from torch's symmetric memory). The exchange PUSHES, and the
// data carries its own arrival mark: a call (same sizes on every rank) has the number e = finished calls + 1, and a
// thread owns 8-byte pieces of the vector. For each of its pieces it
//   1. stores the piece, stamped with e, into inbox[e & 1][my rank] of EVERY rank's buffer (one 16-byte peer store per
//      rank: {4 bytes, e, 4 bytes, e}; the own buffer included);
//   2. polls the same cell of the `world` inboxes of the LOCAL buffer until it carries e, adds the pieces in rank order
//      in f32 and stores the sum to `out`: every rank computes the same sum in the same order - identical bits.
// One NVLink crossing lies on the critical path; there is no flag, no fence and nothing is read remotely. The two
// halves make a second barrier unnecessary: a rank writes half e & 1 of a peer's inbox again only in its call e + 2,
// which it enters after its call e + 1 has received that peer's pieces of call e + 1, sent after the peer finished
// call e. The call number lives in the local buffer and is advanced by the last block of a call to finish, so a
// captured call can be replayed. The wait is bounded: a rank that never arrives makes the others record
// STATUS_WAIT_PEER_TIMEOUT in the device status word and return without writing those pieces of `out`; nothing traps,
// nothing spins forever.
#include "common.cuh"
#include "peer_allreduce.cuh"
#include "runtime.h"

namespace b200q {

struct PeerAllReduceParams {
    PeerExchange px;
    const void* in;
    void* out;
    long long n;  // elements
    unsigned int* status;
};

// `in`, `out` 8-byte aligned, the vector a whole number of 8-byte pieces (the host checks)
template <typename T>
__global__ void __launch_bounds__(PAR_THREADS) peer_allreduce_kernel(const PeerAllReduceParams p) {
    const unsigned int e = par_next_epoch(*reinterpret_cast<volatile unsigned int*>(par_header(p.px) + PAR_EPOCH_ALONE));
    const long long pieces = p.n / Vec8<T>::N;
    const uint2* src = reinterpret_cast<const uint2*>(p.in);
    uint2* dst = reinterpret_cast<uint2*>(p.out);
    const long long step = (long long)gridDim.x * PAR_THREADS;
    const long long first = (long long)blockIdx.x * PAR_THREADS + threadIdx.x;
    // (read past L1: another kernel's CTAs produced the vector)
    for (long long i = first; i < pieces; i += step) peer_push_piece<T>(p.px, PAR_PATH_ALONE, e, i, __ldcg(src + i));
    for (long long i = first; i < pieces; i += step) {
        uint2 sum;
        if (peer_sum_piece<T>(p.px, PAR_PATH_ALONE, e, i, sum, p.status)) dst[i] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) peer_finish_call(p.px, PAR_EPOCH_ALONE, PAR_COUNT_ALONE, e, gridDim.x);
}

long long peer_allreduce_buffer_bytes(long long capacity) { return par_buffer_bytes(capacity); }

int fill_peer_exchange(PeerExchange& px, const void* const* bufs, int rank, int world, long long capacity) {
    if (world < 1 || world > PAR_MAX_WORLD || rank < 0 || rank >= world || capacity <= 0 || capacity % 16 != 0) return B200Q_ERR_INVALID;
    for (int r = 0; r < world; ++r) {
        if (bufs[r] == nullptr || reinterpret_cast<uintptr_t>(bufs[r]) % 16 != 0) return B200Q_ERR_INVALID;
        px.bufs[r] = static_cast<uint8_t*>(const_cast<void*>(bufs[r]));
    }
    px.capacity = capacity;
    px.rank = rank;
    px.world = world;
    return 0;
}

int peer_allreduce(const void* const* bufs, int rank, int world, long long capacity, int elem, const void* in, void* out, long long n,
                   cudaStream_t s) {
    PeerAllReduceParams p{};
    const int rc = fill_peer_exchange(p.px, bufs, rank, world, capacity);
    if (rc != 0) return rc;
    const int esize = elem == ELEM_F32 ? 4 : 2;
    if (n <= 0) return 0;
    if (n * esize > capacity) return B200Q_ERR_TOO_LARGE;
    if ((n * esize) % 16 != 0 || reinterpret_cast<uintptr_t>(in) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0) return B200Q_ERR_UNSUPPORTED;
    p.in = in;
    p.out = out;
    p.n = n;
    p.status = status_ptr();
    // a thread per 8-byte piece, at most one block per SM (every rank derives the same grid from the same sizes)
    const long long pieces = n * esize / 8;
    long long blocks = (pieces + PAR_THREADS - 1) / PAR_THREADS;
    if (blocks > runtime_info().sm_count) blocks = runtime_info().sm_count;
    if (elem == ELEM_F32) peer_allreduce_kernel<float><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_F16) peer_allreduce_kernel<__half><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_BF16) peer_allreduce_kernel<__nv_bfloat16><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else return B200Q_ERR_INVALID;
    return (int)cudaGetLastError();
}

}  // namespace b200q

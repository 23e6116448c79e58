// One-shot sum all-reduce of a small vector over NVLink peer memory: the exchange step after every row-parallel matmul
// of the tensor-parallel decode path (attn_output, ffn_down: [rows, hidden] partial outputs, 16 KB at one row of a
// 70B-class model). Takes the place of the NCCL all-reduce behind the reference's SumAllReduce
// (crates/inference-quant/src/distributed/mod.rs:516-670) where latency, not bandwidth, is the cost: at 8 GPUs a 16 KB
// NCCL all-reduce is a launch of its own of some tens of microseconds, 160 times per token.
//
// Every rank owns one buffer of the same layout (peer_allreduce.cuh), mapped into every other rank's address space (the
// caller provides the mappings; the Python side gets them from torch's symmetric memory). The exchange PUSHES: a call
// on every rank (same sizes everywhere) runs up to seven independent blocks, block i on bytes [i * slot_cap, (i + 1) *
// slot_cap) of the vector:
//   1. e = ++epoch[i]; store the slice of `in` into inbox[i][e & 1][my rank] of EVERY rank's buffer (plain peer stores
//      over NVLink, the own buffer included); system-scope fence;
//   2. write e into arrive[i][my rank] of every peer (release), then wait until every arrive[i][r] of the own buffer has
//      reached e (acquire): all ranks' slices have landed here;
//   3. read the slice from the `world` inboxes of the LOCAL buffer in rank order, add in f32, store to `out`: every rank
//      computes the same sum in the same order, so all ranks hold identical bits.
// One NVLink crossing lies on the critical path (stores, then the flag), and nothing is read remotely. The two halves
// make a second barrier unnecessary: a rank writes half e & 1 of a peer's inbox again only in its call e + 2, which it
// enters after its call e + 1 has seen that peer's signal e + 1, sent after the peer finished reading in call e. A
// slot's inboxes do not depend on the vector's length, so calls of different sizes may follow one another directly.
// Everything is device-side (no host-provided sequence numbers), so a captured call can be replayed.
// The wait is bounded: a rank that never arrives makes the others record STATUS_WAIT_PEER_TIMEOUT in the device status
// word and return without writing `out`; nothing traps, nothing spins forever.
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

// `in`, `out` 16-byte aligned, n a multiple of Vec16<T>::N (the host checks); gridDim.x = ceil(bytes / slot_cap)
template <typename T>
__global__ void __launch_bounds__(PAR_THREADS) peer_allreduce_kernel(const PeerAllReduceParams p) {
    __shared__ unsigned int scratch[2];
    const int slot = blockIdx.x, tid = threadIdx.x;
    const long long units = p.n / Vec16<T>::N;
    const long long per_slot = par_slot_cap(p.px.capacity) / 16;
    const long long u0 = (long long)slot * per_slot;
    const long long nunits = (u0 + per_slot < units ? u0 + per_slot : units) - u0;
    uint8_t* mine = p.px.bufs[p.px.rank];
    if (tid == 0) {
        unsigned int* epoch = reinterpret_cast<unsigned int*>(mine + PAR_EPOCH_OFFSET) + slot;
        const unsigned int e1 = *epoch + 1u;
        *epoch = e1;
        scratch[1] = e1;
    }
    __syncthreads();
    const unsigned int e = scratch[1];
    // 1. this rank's slice into its inbox on every rank (read past L1: other CTAs may have produced it)
    const long long my_inbox = par_inbox_offset(p.px.capacity, slot, e & 1u, p.px.rank);
    const uint4* src = reinterpret_cast<const uint4*>(p.in) + u0;
    for (long long u = tid; u < nunits; u += PAR_THREADS) {
        const uint4 v = __ldcg(src + u);
        for (int r = 0; r < p.px.world; ++r) st_global_16(p.px.bufs[r] + my_inbox + (size_t)u * 16, v);
    }
    __threadfence_system();
    // 2. + 3.
    peer_signal_wait_reduce<T, false>(p.px, slot, e, par_inbox_offset(p.px.capacity, slot, e & 1u, 0), par_slot_cap(p.px.capacity),
                                      reinterpret_cast<uint4*>(p.out) + u0, nunits, tid, PAR_THREADS, p.status, scratch);
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
    // one block per slot the vector reaches, at most seven (slot 7 belongs to the fused launches): every rank derives
    // the same count
    const long long slot_cap = par_slot_cap(capacity);
    long long blocks = (n * esize + slot_cap - 1) / slot_cap;
    if (blocks > PAR_MAX_BLOCKS) return B200Q_ERR_TOO_LARGE;
    if (elem == ELEM_F32) peer_allreduce_kernel<float><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_F16) peer_allreduce_kernel<__half><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_BF16) peer_allreduce_kernel<__nv_bfloat16><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else return B200Q_ERR_INVALID;
    return (int)cudaGetLastError();
}

}  // namespace b200q

// One-shot sum all-reduce of a small vector over NVLink peer memory: the exchange step after every row-parallel matmul
// of the tensor-parallel decode path (attn_output, ffn_down: [rows, hidden] partial outputs, 16 KB at one row of a
// 70B-class model). Takes the place of the NCCL all-reduce behind the reference's SumAllReduce
// (crates/inference-quant/src/distributed/mod.rs:516-670) where latency, not bandwidth, is the cost: at 8 GPUs a 16 KB
// NCCL all-reduce is a launch of its own of some tens of microseconds, 160 times per token.
//
// Every rank owns one buffer of the same layout, mapped into every other rank's address space (the caller provides the
// mappings; the Python side gets them from torch's symmetric memory):
//   bytes [0, 1024)                flags: arrive[slot][source rank] (u32, written by the peers), epoch[slot] at 768,
//                                  the fused launch's CTA arrival counter at 832
//   [1024, 1024 + 2 cap)           staging halves (epoch bit 0 clear / set) of stand-alone calls
//   [1024 + 2 cap, 1024 + 4 cap)   staging halves of the fused matmul + all-reduce launches (slot 7)
// A call on every rank (same sizes everywhere) runs up to seven independent blocks, each on its own slice of the vector:
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

// `in`, `out` 16-byte aligned, n a multiple of Vec16<T>::N (the host checks)
template <typename T>
__global__ void __launch_bounds__(PAR_THREADS) peer_allreduce_kernel(const PeerAllReduceParams p) {
    __shared__ unsigned int scratch[2];
    const long long units = p.n / Vec16<T>::N;
    const long long per_block = (units + gridDim.x - 1) / gridDim.x;
    const long long u0 = blockIdx.x * per_block;
    const long long u1 = u0 + per_block < units ? u0 + per_block : units;
    peer_allreduce_slice<T, false>(p.px, PAR_HEADER_BYTES, blockIdx.x, p.in, p.out, u0, u1, threadIdx.x, PAR_THREADS, p.status, scratch);
}

long long peer_allreduce_buffer_bytes(long long capacity) { return PAR_HEADER_BYTES + 4 * capacity; }

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
    // one block per 8 KB, at most seven (slot 7 belongs to the fused launches): every rank derives the same count
    long long blocks = (n * esize + 8191) / 8192;
    if (blocks > PAR_MAX_BLOCKS) blocks = PAR_MAX_BLOCKS;
    if (elem == ELEM_F32) peer_allreduce_kernel<float><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_F16) peer_allreduce_kernel<__half><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else if (elem == ELEM_BF16) peer_allreduce_kernel<__nv_bfloat16><<<(unsigned)blocks, PAR_THREADS, 0, s>>>(p);
    else return B200Q_ERR_INVALID;
    return (int)cudaGetLastError();
}

}  // namespace b200q

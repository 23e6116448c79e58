// Decode-time GEMV: dst[b][row] = sum_k W[row][k] * x[b][k] for packed Q8_0 / Q4_K / Q6_K weights in their GGUF
// layout and 1..8 activation rows, replacing the reference's `mmvq_gguf_<type>_<dst>_plain_cuda{1..8}`
// (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:688-759, launcher :1762-1834).
//
// Design (HBM-bound; no tensor cores):
//  * Weight rows are contiguous, so the matrix is one byte stream. One persistent CTA per SM owns a contiguous range
//    of rows and streams it through a ring of shared-memory stages with 1-D bulk (TMA) copies issued by one producer
//    thread; full/empty mbarriers hand stages to sixteen consumer warps. Many KB per SM stay in flight with no
//    registers spent on it, and the 2-byte-aligned Q6_K / Q8_0 blocks need no aligned global loads.
//  * A row is cut into work items of 128 values (half a superblock, or four Q8_0 blocks); a warp covers a
//    4096-wide row alone, wider rows are shared by several warps. Each lane owns the same item slots for the whole
//    kernel, so for 1-2 activation rows its quantized activations stay in registers; larger batches read them from
//    shared memory, where they are staged once per CTA as 80-byte records per 64 values
//    {i8 q[64]; f32 d[2]; f32 d*sum(q)[2]} (the 80-byte stride makes the 128-bit reads conflict-free).
//    Activations come either from Q8_1 blocks written by the quantize launcher (the reference's two-launch protocol)
//    or straight from bf16/f16/f32 rows, quantized in the prologue (one launch).
//  * Consumers unpack nibbles and 6-bit scales in registers, use dp4a on 4 packed int8, fold the sub-block scales
//    as integers and the block scales in f32, and reduce with warp shuffles. Warps run independently (no CTA-wide
//    barrier per stage); a row shared by several warps is combined by whichever of them arrives last, adding the
//    partial sums in a fixed order, so results are deterministic.
//  * Every mbarrier wait is bounded and reports through the device status word.
#pragma once
#include <type_traits>

#include "common.cuh"
#include "peer_allreduce.cuh"
#include "runtime.h"

namespace b200q {

constexpr int GEMV_CONSUMER_WARPS = 16;
constexpr int GEMV_CONSUMER_THREADS = GEMV_CONSUMER_WARPS * 32;
constexpr int GEMV_THREADS = GEMV_CONSUMER_THREADS + 32;
constexpr int GEMV_MAX_STAGES = 16;
constexpr int GEMV_BARRIER_BYTES = 2 * GEMV_MAX_STAGES * 8;  // full[] and empty[]
constexpr int ACT_REC_BYTES = 80;  // i8 q[64]; f32 d[2]; f32 ds[2]

enum ActMode : int { ACT_Q8_1 = 0, ACT_RAW_Q8_1 = 1, ACT_RAW_CPU = 2 };

// The matrix the next launch on the stream will read (runtime.h: WeightSuccessor), cut the way that launch will cut
// it: CTA c of that launch owns units [c * q + min(c, r), ...) of unit_bytes each. Each CTA of THIS launch asks L2 for
// the first `bytes` of the range CTA c of the next launch will stream first. w == nullptr: nothing registered.
struct NextPrefetch {
    const uint8_t* w;
    long long total_bytes;  // size of the successor's packed rows, rounded down to 16
    int unit_bytes, units_per_cta, units_extra, grid;
    int bytes;              // per CTA, multiple of 16
};

__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}

// Called by the producer thread once its last weight copy is on its way: the requests queue behind this CTA's own
// copies, so they run as those drain - through the tail of this grid and the launch gap after it.
__device__ __forceinline__ void prefetch_successor(const NextPrefetch& n, int cta) {
    if (n.w == nullptr || cta >= n.grid) return;
    const long long unit0 = (long long)cta * n.units_per_cta + min(cta, n.units_extra);
    const long long units = n.units_per_cta + (cta < n.units_extra ? 1 : 0);
    const long long off = unit0 * n.unit_bytes;
    long long len = units * n.unit_bytes;
    if (off + len > n.total_bytes) len = n.total_bytes - off;
    if (len > n.bytes) len = n.bytes;
    len &= ~15LL;
    for (long long o = 0; o < len; o += 16384) {
        const long long chunk = len - o < 16384 ? len - o : 16384;
        bulk_prefetch_l2(n.w + off + o, (uint32_t)chunk);
    }
}

struct GemvParams {
    const uint8_t* w;   // packed weights, row-major blocks, 16-byte aligned, >= 16 readable bytes after the end
    const void* act;    // Q8_1 blocks [B][stride_act] (ACT_Q8_1) or raw rows [B][stride_act elements]
    void* dst;          // [B][stride_dst]
    int K, N;
    int stride_act;
    int stride_dst;
    int row_bytes;
    int rows_per_stage;  // R: rows one stage holds (multiple of row_align and of the number of row groups)
    int warps_per_row;   // WPR: power of two <= 16; 16 / WPR row groups work on different rows at once
    int log2_wpr;        // shifts instead of divisions in the kernel: WPR = 1 << log2_wpr,
    int log2_islots;     // islots (lanes that share a row inside a warp: items rounded up to a power of two, <= 32)
    int items_per_lane;  // IPL: item slots of one lane: item = (warp % WPR) * 32 + lane + j * 32 * WPR, j < IPL
    int row_align;       // rows per 16-byte-aligned unit of the byte stream
    int units_per_cta;   // CTA c owns units [c * q + min(c, r), ...) with q = units_per_cta, r = units_extra
    int units_extra;
    int nstages;
    int stage_bytes;     // multiple of 128
    int act_bytes;       // bytes of activation records
    int use_pdl;
    int act_vec;         // raw activations: rows are 16-byte aligned
    unsigned int* status;  // device status word
    unsigned long long* trace;  // optional: 16 timestamps (ns) written by the first and by the last CTA, or nullptr
    PeerExchange px;     // px.world > 1: every CTA exchanges its rows of dst with the other ranks and stores their sum
    int ar_rows;         // fused exchange: rows per activation row of the CTA's output staging area (a multiple of row_align)
    int ar_offset;       // and its offset in dynamic shared memory
    NextPrefetch next;   // the registered successor matrix, or w == nullptr
};

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Launch timelines are a build option (-DB200Q_GEMV_TRACE=1): fifteen timestamp sites are a few hundred instructions in
// every kernel, and the decode chain is sensitive to the size of its kernels' code.
#ifndef B200Q_GEMV_TRACE
#define B200Q_GEMV_TRACE 0
#endif
#if B200Q_GEMV_TRACE
#define GEMV_TRACE_ANY(slot)                                                                               \
    do {                                                                                                   \
        if (p.trace != nullptr && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))                        \
            p.trace[(blockIdx.x == 0 ? 0 : 16) + (slot)] = global_timer_ns();                              \
    } while (0)
#define GEMV_TRACE(slot)                                                                                   \
    do {                                                                                                   \
        if (p.trace != nullptr && tid == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))            \
            p.trace[(blockIdx.x == 0 ? 0 : 16) + (slot)] = global_timer_ns();                               \
    } while (0)
#else
#define GEMV_TRACE_ANY(slot) do { } while (0)
#define GEMV_TRACE(slot) do { } while (0)
#endif

// ---------------------------------------------------------------------------------------------
// Activation staging (generic stores into shared memory; read back with explicit shared loads)
// ---------------------------------------------------------------------------------------------

// The first unit of activation data of each thread, loaded at the very top of the kernel: a Q8_1 block (9 words) or
// 8 raw values.
template <int ACT, typename act_t> struct ActPrefetch;
template <typename act_t> struct ActPrefetch<ACT_Q8_1, act_t> {
    uint32_t v[9];
    __device__ __forceinline__ void issue(const void* act, int B, int K, int stride_blocks, bool, int tid) {
        const int nblk = K / 32;
        if (tid < B * nblk) {
            const int b = tid / nblk, kb = tid - b * nblk;
            const uint32_t* src =
                reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(act) + ((size_t)b * stride_blocks + kb) * Q8_1_BYTES);
#pragma unroll
            for (int j = 0; j < 9; ++j) v[j] = src[j];
        }
    }
};

// From Q8_1 blocks: one thread per 32-value block.
template <int B, typename Pre>
__device__ __forceinline__ void stage_acts_q8_1(uint8_t* acts, const uint8_t* vy, int K, int stride_blocks, int tid,
                                                int nthreads, const Pre& pre) {
    const int nblk = K / 32;
    const int nrec = K / 64;
    for (int i = tid; i < B * nblk; i += nthreads) {
        const int b = i / nblk, kb = i - b * nblk;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(vy + ((size_t)b * stride_blocks + kb) * Q8_1_BYTES);
        uint8_t* rec = acts + ((size_t)b * nrec + (kb >> 1)) * ACT_REC_BYTES;
        const int h = kb & 1;
        uint32_t v[9];
        if (i == tid) {
#pragma unroll
            for (int j = 0; j < 9; ++j) v[j] = pre.v[j];
        } else {
#pragma unroll
            for (int j = 0; j < 9; ++j) v[j] = src[j];
        }
        int sum = 0;
        uint32_t* qdst = reinterpret_cast<uint32_t*>(rec + 32 * h);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            qdst[j] = v[1 + j];
            sum = dp4a_ss(0x01010101u, v[1 + j], sum);
        }
        const float d = half_bits_to_float(v[0]);
        reinterpret_cast<float*>(rec + 64)[h] = d;
        reinterpret_cast<float*>(rec + 72)[h] = d * (float)sum;
    }
}

// Eight consecutive activations as f32. `vec`: the address is 16-byte aligned, so 128-bit loads are used.
template <typename src_t>
__device__ __forceinline__ void load8(const src_t* p, bool vec, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, bool vec, float (&v)[8]) {
    if (vec) {
        const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = p[j];
    }
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, bool vec, float (&v)[8]) {
    if (vec) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __half22float2(h[j]);
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __half2float(p[j]);
    }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, bool vec, float (&v)[8]) {
    if (vec) {
        const uint4 u = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            v[2 * j] = f.x;
            v[2 * j + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __bfloat162float(p[j]);
    }
}

// Raw activations: up to PRE_UNITS chunks of 8 values per thread, kept as raw bits so that nothing waits for the
// loads until the values are used.
constexpr int PRE_UNITS = 4;
template <int ACT, typename act_t> struct ActPrefetch {
    static constexpr int WORDS = sizeof(act_t) * 2;  // 32-bit words per chunk of 8 values
    uint32_t raw[PRE_UNITS][WORDS];
    __device__ __forceinline__ void issue(const void* act, int B, int K, int stride_elems, bool vec, int tid) {
        const int chunks = K / 8;
#pragma unroll
        for (int u = 0; u < PRE_UNITS; ++u) {
            const int i = tid + u * GEMV_CONSUMER_THREADS;
            if (i < B * chunks) {
                const int b = B == 1 ? 0 : i / chunks, c = i - b * chunks;  // (no division on the single-row path)
                const act_t* src = reinterpret_cast<const act_t*>(act) + (size_t)b * stride_elems + 8 * c;
                if (vec) {
#pragma unroll
                    for (int q = 0; q < WORDS / 4; ++q) {
                        const uint4 t = reinterpret_cast<const uint4*>(src)[q];
                        raw[u][4 * q] = t.x; raw[u][4 * q + 1] = t.y; raw[u][4 * q + 2] = t.z; raw[u][4 * q + 3] = t.w;
                    }
                } else if (sizeof(act_t) == 4) {
#pragma unroll
                    for (int q = 0; q < WORDS; ++q) raw[u][q] = reinterpret_cast<const uint32_t*>(src)[q];
                } else {
#pragma unroll
                    for (int q = 0; q < WORDS; ++q) {
                        const unsigned short lo = reinterpret_cast<const unsigned short*>(src)[2 * q];
                        const unsigned short hi = reinterpret_cast<const unsigned short*>(src)[2 * q + 1];
                        raw[u][q] = (uint32_t)lo | ((uint32_t)hi << 16);
                    }
                }
            }
        }
    }
    __device__ __forceinline__ void get(int u, float (&v)[8]) const;
};
template <> __device__ __forceinline__ void ActPrefetch<ACT_RAW_Q8_1, float>::get(int u, float (&v)[8]) const {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(raw[u][j]);
}
template <> __device__ __forceinline__ void ActPrefetch<ACT_RAW_CPU, float>::get(int u, float (&v)[8]) const {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(raw[u][j]);
}
#define B200Q_PREFETCH_GET16(MODE, T, CONV2, T2)                                                        \
    template <> __device__ __forceinline__ void ActPrefetch<MODE, T>::get(int u, float (&v)[8]) const { \
        _Pragma("unroll") for (int j = 0; j < 4; ++j) {                                                 \
            const float2 f = CONV2(*reinterpret_cast<const T2*>(&raw[u][j]));                           \
            v[2 * j] = f.x;                                                                             \
            v[2 * j + 1] = f.y;                                                                         \
        }                                                                                               \
    }
B200Q_PREFETCH_GET16(ACT_RAW_Q8_1, __half, __half22float2, __half2)
B200Q_PREFETCH_GET16(ACT_RAW_CPU, __half, __half22float2, __half2)
B200Q_PREFETCH_GET16(ACT_RAW_Q8_1, __nv_bfloat16, __bfloat1622float2, __nv_bfloat162)
B200Q_PREFETCH_GET16(ACT_RAW_CPU, __nv_bfloat16, __bfloat1622float2, __nv_bfloat162)

// roundf(v / d) with the IEEE division, kept out of line: the quantizer below needs it for the few values whose quotient
// lies next to a rounding boundary, and eight inlined copies would sit in every launch's instruction stream
static __device__ __noinline__ int round_div_exact(float v, float d) { return (int)roundf(v / d); }

// From raw rows, quantized here. Each thread takes 8 consecutive values, so 4 lanes share a 32-value block and a warp
// covers 256 values.
//   ACT_RAW_Q8_1: the decode quantizer's arithmetic (d = amax / 127 rounded to f16, q = roundf(x / d)): identical to
//                 running launch_mmvq_gguf_quantize_q8_1_* first.
//   ACT_RAW_CPU:  the reference CPU path's activation format for the weight type: Q8_K for Q4_K / Q6_K (one f32 scale
//                 per 256 values, iscale = -127 / max, crates/inference-tensor/src/quantized/k_quants.rs:2721-2760) and
//                 Q8_0 for Q8_0 (per 32, f16 scale, q = round(x * (1 / d)), quantized/mod.rs:43-56). The integer dot
//                 products then equal the CPU path's exactly.
template <int B, typename src_t, int TYPE, int MODE, typename Pre>
__device__ __forceinline__ void stage_acts_raw(uint8_t* acts, const src_t* x, int K, int stride_elems, bool vec, int tid,
                                               int nthreads, const Pre& pre) {
    const int chunks = K / 8;
    const int nrec = K / 64;
    const int lane = tid & 31;
    constexpr bool PER_256 = (MODE == ACT_RAW_CPU) && (TYPE != TYPE_Q8_0);
    // The shuffles below name the whole warp: a shuffle whose mask differs between the lanes of one instruction is
    // carried out one mask after the other and costs hundreds of cycles a piece, four times per chunk. So the loop's
    // trip count is the same for all lanes of a warp (lanes past the end work on zeros and store nothing).
    constexpr unsigned gmask = 0xffffffffu;
    const int total = B * chunks;
    int u = 0;  // which of this thread's chunks
    // (One chunk after the other: processing the chunks loaded ahead side by side shortens a single launch by 3-5 % and
    // makes the kernel's code larger; in the decode chain, where three kernels alternate, that cost 10 %.)
    for (int i = tid; i - lane < total; i += nthreads, ++u) {
        const bool valid = i < total;
        // integer divisions are dozens of dependent instructions on a path every launch runs exactly once
        const int b = B == 1 ? 0 : (valid ? i / chunks : 0), c = B == 1 ? i : i - b * chunks;
        float v[8];
        if (u == 0) pre.get(0, v);
        else if (u == 1) pre.get(1, v);
        else if (u == 2) pre.get(2, v);
        else if (u == 3) pre.get(3, v);
        else if (valid) load8<src_t>(x + (size_t)b * stride_elems + 8 * c, vec, v);
        if (!valid) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = 0.0f;
        }
        int q[8];
        float d_used;
        if (PER_256) {
            float amax = 0.0f, mx = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (amax < fabsf(v[j])) { amax = fabsf(v[j]); mx = v[j]; }
            int who = lane;
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {  // the first value of largest magnitude, as the CPU loop finds it
                const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
                const float om = __shfl_xor_sync(0xffffffffu, mx, off);
                const int ow = __shfl_xor_sync(0xffffffffu, who, off);
                if (oa > amax || (oa == amax && ow < who)) { amax = oa; mx = om; who = ow; }
            }
            if (amax == 0.0f) {
#pragma unroll
                for (int j = 0; j < 8; ++j) q[j] = 0;
                d_used = 0.0f;
            } else {
                const float iscale = -127.0f / mx;
#pragma unroll
                for (int j = 0; j < 8; ++j) q[j] = (int)fminf(fmaxf(roundf(iscale * v[j]), -128.0f), 127.0f);
                d_used = 1.0f / iscale;
            }
        } else {
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
            amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 2));
            // amax / 127 correctly rounded without the division routine: multiply by the rounded reciprocal, then one
            // residual correction (exact for every finite amax whose quotient is a normal number; smaller ones take the
            // division, which then also matches)
            float d = amax * 0.007874015718698502f;
            d = fmaf(fmaf(-127.0f, d, amax), 0.007874015718698502f, d);
            if (amax < 1e-30f) d = amax / 127.0f;
            if (MODE == ACT_RAW_CPU) {
                const float id = d != 0.0f ? 1.0f / d : 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) q[j] = (int)roundf(v[j] * id);
            } else {
                // roundf(x / d) without eight IEEE divisions. x * (1 / d) + 1.5 * 2^23 leaves the nearest integer in the
                // low mantissa bits (its low byte is the quant as stored) and, minus the constant, as a float; the exact
                // remainder x - d * q then tells how far the true quotient is from q. Where that is under 0.4999 the
                // correctly rounded quotient (within 4e-6 of the true one for |q| < 128) rounds to q as well; the others
                // (one value in 5000, and every exact tie) are decided by the division itself, out of line.
                const float rcp = amax == 0.0f ? 0.0f : __frcp_rn(d);
                const float lim = 0.4999f * d;
                unsigned near_half = 0u;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float t = fmaf(v[j], rcp, 12582912.0f);
                    const float rem = fmaf(-d, t - 12582912.0f, v[j]);
                    q[j] = (int)__float_as_uint(t);  // only the low byte is used
                    near_half |= (fabsf(rem) > lim) ? (1u << j) : 0u;
                }
                // a lane rarely flags more than one of its values, so the warp goes round once per flagged value of its
                // worst lane, not once per position any lane flagged (the block's warps meet at a barrier after this,
                // so the slowest warp sets the time)
                while (near_half != 0u) {
                    const int j = __ffs(near_half) - 1;
                    near_half &= near_half - 1u;
                    float vj = v[0];
#pragma unroll
                    for (int t = 1; t < 8; ++t) vj = j == t ? v[t] : vj;
                    const int r = round_div_exact(vj, d);
#pragma unroll
                    for (int t = 0; t < 8; ++t) q[t] = j == t ? r : q[t];
                }
            }
            d_used = __half2float(__float2half_rn(d));
        }
        // the low bytes four to a word, and the chunk's sum from the bytes as stored
        const uint32_t w0 = __byte_perm(__byte_perm((uint32_t)q[0], (uint32_t)q[1], 0x0040), __byte_perm((uint32_t)q[2], (uint32_t)q[3], 0x0040), 0x5410);
        const uint32_t w1 = __byte_perm(__byte_perm((uint32_t)q[4], (uint32_t)q[5], 0x0040), __byte_perm((uint32_t)q[6], (uint32_t)q[7], 0x0040), 0x5410);
        int sum = __dp4a((int)w0, 0x01010101, __dp4a((int)w1, 0x01010101, 0));
        sum += __shfl_xor_sync(gmask, sum, 1);
        sum += __shfl_xor_sync(gmask, sum, 2);
        if (!valid) continue;
        uint8_t* rec = acts + ((size_t)b * nrec + (c >> 3)) * ACT_REC_BYTES;
        const int h = (c >> 2) & 1;
        *reinterpret_cast<uint2*>(rec + 32 * h + 8 * (c & 3)) = make_uint2(w0, w1);
        if ((c & 3) == 0) {
            reinterpret_cast<float*>(rec + 64)[h] = d_used;
            reinterpret_cast<float*>(rec + 72)[h] = d_used * (float)sum;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Per-type work items: one item = 128 consecutive values of a row (half a superblock; four Q8_0 blocks), matched by
// activation records 2*item and 2*item+1. All addresses are 32-bit shared-space addresses.
//   Weights<TYPE>::load(row_addr, item)   reads one item of a weight row from a stage
//   Acts<TYPE>::load(act_row_addr, item)  reads the matching quantized activations of one activation row
//   dot(W, A)                             their contribution to the output, in f32
// ---------------------------------------------------------------------------------------------
template <int TYPE> struct Weights;
template <int TYPE> struct Acts;

// two 80-byte activation records in registers: 128 int8 and, per 32 of them, d and d * sum(q)
struct ActPair {
    uint32_t q[32];
    float d[4], ds[4];
    __device__ __forceinline__ void load(uint32_t act_row, int item) {
        const uint32_t rec = act_row + (uint32_t)item * (2 * ACT_REC_BYTES);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t a = rec + r * ACT_REC_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = lds128(a + 16 * j);
                q[16 * r + 4 * j + 0] = v.x; q[16 * r + 4 * j + 1] = v.y; q[16 * r + 4 * j + 2] = v.z; q[16 * r + 4 * j + 3] = v.w;
            }
            const uint4 f = lds128(a + 64);
            d[2 * r] = __uint_as_float(f.x); d[2 * r + 1] = __uint_as_float(f.y);
            ds[2 * r] = __uint_as_float(f.z); ds[2 * r + 1] = __uint_as_float(f.w);
        }
    }
};

// ---- Q4_K: item (s, h) = chunks c = 2h, 2h+1 of superblock s: 64 bytes of nibbles; in chunk c the low nibbles are
// sub-block 2c and the high nibbles sub-block 2c+1.
template <> struct Weights<TYPE_Q4_K> {
    uint32_t w[16];
    uint32_t sc4, m4;  // the four 6-bit scales / mins of sub-blocks 4h .. 4h+3, one per byte
    float d, dmin;
    __device__ __forceinline__ void load(uint32_t row_addr, int item) {
        const int s = item >> 1, h = item & 1;
        const uint32_t sb = row_addr + s * Q4_K_BYTES;
        const uint4 hdr = lds128(sb);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 v = lds128(sb + 16 + 64 * h + 16 * j);
            w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
        // 6-bit scales and mins (crates/inference-tensor/src/quantized/utils.rs:119-129), four at a time
        // (both forms computed and selected: h alternates between neighbouring lanes, and a branch would split every warp)
        const uint32_t sc_lo = hdr.y & 0x3f3f3f3fu, m_lo = hdr.z & 0x3f3f3f3fu;
        const uint32_t sc_hi = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
        const uint32_t m_hi = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
        sc4 = h == 0 ? sc_lo : sc_hi;
        m4 = h == 0 ? m_lo : m_hi;
        d = half_bits_to_float(hdr.x);
        dmin = half_bits_to_float(hdr.x >> 16);
    }
};
template <> struct Acts<TYPE_Q4_K> : ActPair {};
__device__ __forceinline__ float dot(const Weights<TYPE_Q4_K>& W, const ActPair& A) {
    float accd = 0.0f, accm = 0.0f;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
        int dl0 = 0, dl1 = 0, dh0 = 0, dh1 = 0;  // two chains per half keep the dp4a pipe busy
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            dl0 = dp4a_us(W.w[8 * cc + j] & 0x0f0f0f0fu, A.q[16 * cc + j], dl0);
            dl1 = dp4a_us(W.w[8 * cc + 4 + j] & 0x0f0f0f0fu, A.q[16 * cc + 4 + j], dl1);
            dh0 = dp4a_us(W.w[8 * cc + j] & 0xf0f0f0f0u, A.q[16 * cc + 8 + j], dh0);       // 16 * high nibble
            dh1 = dp4a_us(W.w[8 * cc + 4 + j] & 0xf0f0f0f0u, A.q[16 * cc + 12 + j], dh1);
        }
        // one byte of the packed scales / mins each (a byte permute: one instruction instead of shift + mask)
        const int sc_lo = (int)__byte_perm(W.sc4, 0u, 0x4440u + 2 * cc), sc_hi = (int)__byte_perm(W.sc4, 0u, 0x4441u + 2 * cc);
        // a min (<= 63) as a float: its byte dropped into the low byte of 2^23 + 2^22 (exact), minus that constant
        const float m_lo = __uint_as_float(__byte_perm(W.m4, 0x4B400000u, 0x7650u + 2 * cc)) - 12582912.0f;
        const float m_hi = __uint_as_float(__byte_perm(W.m4, 0x4B400000u, 0x7651u + 2 * cc)) - 12582912.0f;
        // integer scale folding: |sc * dot| <= 63 * 32 * 15 * 127 < 2^22
        accd += A.d[2 * cc] * int_to_float_small(sc_lo * (dl0 + dl1));
        accd += A.d[2 * cc + 1] * int_to_float_small(sc_hi * ((dh0 + dh1) >> 4));
        accm += m_lo * A.ds[2 * cc] + m_hi * A.ds[2 * cc + 1];
    }
    return W.d * accd - W.dmin * accm;
}

// Reads N consecutive 32-bit words starting at the 2-byte-aligned shared address a.
template <int N>
__device__ __forceinline__ void lds_words_u16aligned(uint32_t a, uint32_t (&out)[N]) {
    const uint32_t shift = (a & 2u) * 8u;
    const uint32_t base = a & ~3u;
    uint32_t prev = lds32(base);
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = lds32(base + 4 * (i + 1));
        out[i] = __funnelshift_r(prev, next, shift);
        prev = next;
    }
}

// ---- Q6_K: item (s, n) = half n of superblock s: ql[64n..], qh[32n..], scales[8n..]; byte l of the half holds
// one value of each of the four 32-value quarters (crates/inference-tensor/src/quantized/k_quants.rs:2661-2677).
// Weights are rebuilt as 4 * (q - 32) in a signed byte: ((q ^ 32) << 2) reinterpreted, so no subtraction and one
// signed dp4a; the factor 4 is folded into d.
template <> struct Weights<TYPE_Q6_K> {
    uint32_t ql[16], qh[8], scw[2];
    float d;
    __device__ __forceinline__ void load(uint32_t row_addr, int item) {
        const int s = item >> 1, n = item & 1;
        const uint32_t sb = row_addr + s * Q6_K_BYTES;
        lds_words_u16aligned<16>(sb + 64 * n, ql);
        lds_words_u16aligned<8>(sb + 128 + 32 * n, qh);
        lds_words_u16aligned<2>(sb + 192 + 8 * n, scw);
        d = half_bits_to_float(lds16(sb + 208)) * 0.25f;
    }
};
// the 128 activations of half n in order: quarter qd = values 32*qd .. 32*qd+31 = words 8*qd .. 8*qd+7
template <> struct Acts<TYPE_Q6_K> {
    uint32_t q[32];
    float d[4];
    __device__ __forceinline__ void load(uint32_t act_row, int item) {
        const uint32_t rec = act_row + (uint32_t)item * (2 * ACT_REC_BYTES);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t a = rec + r * ACT_REC_BYTES;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint4 v = lds128(a + 16 * j);
                q[16 * r + 4 * j + 0] = v.x; q[16 * r + 4 * j + 1] = v.y; q[16 * r + 4 * j + 2] = v.z; q[16 * r + 4 * j + 3] = v.w;
            }
            const uint2 f = lds64(a + 64);
            d[2 * r] = __uint_as_float(f.x); d[2 * r + 1] = __uint_as_float(f.y);
        }
    }
};
__device__ __forceinline__ float dot_q6k(const Weights<TYPE_Q6_K>& W, const uint32_t (&aq)[32], const float (&ad)[4]) {
    int acc[4][2];
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) acc[qd][0] = acc[qd][1] = 0;
#pragma unroll
    for (int t = 0; t < 8; ++t) {  // bytes l = 4t .. 4t+3 of the half; 16-value group g = t / 4
        const uint32_t la = W.ql[t], lb = W.ql[8 + t], h = W.qh[t];
        const uint32_t w0 = ((la << 2) & 0x3c3c3c3cu) | (((h << 6) & 0xc0c0c0c0u) ^ 0x80808080u);
        const uint32_t w1 = ((lb << 2) & 0x3c3c3c3cu) | (((h << 4) & 0xc0c0c0c0u) ^ 0x80808080u);
        const uint32_t w2 = ((la >> 2) & 0x3c3c3c3cu) | (((h << 2) & 0xc0c0c0c0u) ^ 0x80808080u);
        const uint32_t w3 = ((lb >> 2) & 0x3c3c3c3cu) | ((h & 0xc0c0c0c0u) ^ 0x80808080u);
        const int g = t >> 2;
        acc[0][g] = dp4a_ss(w0, aq[t], acc[0][g]);
        acc[1][g] = dp4a_ss(w1, aq[8 + t], acc[1][g]);
        acc[2][g] = dp4a_ss(w2, aq[16 + t], acc[2][g]);
        acc[3][g] = dp4a_ss(w3, aq[24 + t], acc[3][g]);
    }
    float part = 0.0f;
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {  // scales[8n + 2*qd + g]
        const uint32_t word = qd < 2 ? W.scw[0] : W.scw[1];
        const int s0 = (int)(int8_t)((word >> (16 * (qd & 1))) & 0xffu);
        const int s1 = (int)(int8_t)((word >> (16 * (qd & 1) + 8)) & 0xffu);
        part += ad[qd] * (float)(s0 * acc[qd][0] + s1 * acc[qd][1]);
    }
    return W.d * part;
}

__device__ __forceinline__ float dot(const Weights<TYPE_Q6_K>& W, const Acts<TYPE_Q6_K>& A) { return dot_q6k(W, A.q, A.d); }
__device__ __forceinline__ float dot(const Weights<TYPE_Q6_K>& W, const ActPair& A) { return dot_q6k(W, A.q, A.d); }

// ---- Q8_0: item = four 34-byte blocks.
template <> struct Weights<TYPE_Q8_0> {
    uint32_t q[32];
    float d[4];
    __device__ __forceinline__ void load(uint32_t row_addr, int item) {
        uint32_t w[34];
        lds_words_u16aligned<34>(row_addr + (uint32_t)item * (4 * Q8_0_BYTES), w);  // 136 bytes
        // block b starts at byte 34 b: f16 d, then 32 quants
        d[0] = half_bits_to_float(w[0]);
        d[1] = half_bits_to_float(w[8] >> 16);
        d[2] = half_bits_to_float(w[17]);
        d[3] = half_bits_to_float(w[25] >> 16);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            q[j] = __funnelshift_r(w[j], w[j + 1], 16);             // bytes 2 .. 33
            q[8 + j] = w[9 + j];                                    // bytes 36 .. 67
            q[16 + j] = __funnelshift_r(w[17 + j], w[18 + j], 16);  // bytes 70 .. 101
            q[24 + j] = w[26 + j];                                  // bytes 104 .. 135
        }
    }
};
template <> struct Acts<TYPE_Q8_0> : ActPair {};
__device__ __forceinline__ float dot(const Weights<TYPE_Q8_0>& W, const ActPair& A) {
    float part = 0.0f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        int v0 = 0, v1 = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            v0 = dp4a_ss(W.q[8 * b + j], A.q[8 * b + j], v0);
            v1 = dp4a_ss(W.q[8 * b + 4 + j], A.q[8 * b + 4 + j], v1);
        }
        part += W.d[b] * (A.d[b] * int_to_float_small(v0 + v1));
    }
    return part;
}

// Fused exchange, called by the consumer threads of a CTA whose rows [row0, row1) of the [B][N] output sit in shared
// memory (`stage`, `stage_rows` entries per activation row): 8-byte pieces of the output (row0 and the row count are whole
// pieces: the planner aligned the CTA's row range), each stamped with the call number and stored into this rank's inbox
// on every rank, then summed from the local inboxes as the peers' CTAs deliver theirs, and written to `dst`. No fence,
// no flag, no last CTA: one NVLink crossing after the slowest rank's CTA has finished its rows (peer_allreduce.cuh).
template <typename dst_t, int B>
__device__ __forceinline__ void exchange_cta_rows(const PeerExchange& px, const dst_t* stage, int stage_rows, int row0, int row1, int N,
                                                  void* dst, unsigned int* status, int tid, unsigned int epoch) {
    named_bar_sync(1, GEMV_CONSUMER_THREADS);  // the CTA's outputs are in shared memory
    constexpr int PIECE = 8 / (int)sizeof(dst_t);
    const int pieces_per_row = (row1 - row0) / PIECE;
    const int total = B * pieces_per_row;
    for (int i = tid; i < total; i += GEMV_CONSUMER_THREADS) {
        const int b = B == 1 ? 0 : i / pieces_per_row, pr = i - b * pieces_per_row;
        const uint2 mine = *reinterpret_cast<const uint2*>(stage + b * stage_rows + pr * PIECE);
        peer_push_piece<dst_t>(px, PAR_PATH_FUSED, epoch, ((long long)b * N + row0) / PIECE + pr, mine);
    }
    for (int i = tid; i < total; i += GEMV_CONSUMER_THREADS) {
        const int b = B == 1 ? 0 : i / pieces_per_row, pr = i - b * pieces_per_row;
        const long long piece = ((long long)b * N + row0) / PIECE + pr;
        uint2 sum;
        if (peer_sum_piece<dst_t>(px, PAR_PATH_FUSED, epoch, piece, sum, status)) reinterpret_cast<uint2*>(dst)[piece] = sum;
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    if (tid == 0) peer_finish_call(px, PAR_EPOCH_FUSED, PAR_COUNT_FUSED, epoch, gridDim.x);
}

// ---------------------------------------------------------------------------------------------
// The kernel. NREG = item slots per lane whose activations live in registers (0: read from shared memory each time).
//
// Lanes and items: a row has K / 128 items. With >= 32 items a row is shared by WPR warps (slice = warp % WPR) and a
// lane owns items slice*32 + lane + j*32*WPR, j < IPL. With fewer, a warp works on 32 / islots rows at once
// (islots = items rounded up to a power of two): lane = rsub * islots + item.
// ---------------------------------------------------------------------------------------------
// AR: the variant whose CTAs exchange their rows of the output with the other tensor-parallel ranks and store the sum (its
// own instantiation, so that the plain kernel carries none of it)
template <int TYPE, int B, typename dst_t, int ACT, typename act_t, int NREG, bool AR = false>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_staged_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GEMV_MAX_STAGES;
    uint8_t* acts = smem + GEMV_BARRIER_BYTES;
    const int S = p.nstages, R = p.rows_per_stage, WPR = p.warps_per_row, IPL = p.items_per_lane;
    // cross-warp combine (WPR > 1): per stage and row, WPR partial sums per activation row and an arrival counter
    float* partial = reinterpret_cast<float*>(acts + p.act_bytes);  // [S][R][WPR][B]
    const int partial_floats = WPR > 1 ? S * R * WPR * B : 0;
    int* counters = reinterpret_cast<int*>(partial + partial_floats);  // [S][R]
    const int counter_ints = WPR > 1 ? S * R : 0;
    uint8_t* ring = acts + p.act_bytes + (((partial_floats + counter_ints) * 4 + 127) & ~127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    GEMV_TRACE(0);
    // Under programmatic dependent launch this grid may start while the previous one is still running (on the SMs that
    // grid has left): barrier set-up and the weight stream do not depend on it and go ahead; only the consumers wait
    // for it - after the CTA-wide barrier below, so that they do not hold the producer back - before they touch the
    // activations it wrote.
    if (p.use_pdl) grid_launch_dependents();  // and the grid after this one may start its own set-up
    // Without it, the first activation loads go out before anything else: issued after the weight stream has started
    // they would queue behind megabytes of bulk copies.
    ActPrefetch<ACT, act_t> pre;
    if (!p.use_pdl && warp != GEMV_CONSUMER_WARPS) pre.issue(p.act, B, p.K, p.stride_act, p.act_vec != 0, tid);

    // this CTA's rows: a contiguous run of 16-byte-aligned units, sizes differing by at most one unit
    const int cta = blockIdx.x;
    const int unit0 = cta * p.units_per_cta + min(cta, p.units_extra);
    const int row0 = unit0 * p.row_align;
    int row1 = (unit0 + p.units_per_cta + (cta < p.units_extra ? 1 : 0)) * p.row_align;
    if (row1 > p.N) row1 = p.N;
    if (row1 < row0) row1 = row0;  // the stages of this CTA are the row offsets row0, row0 + R, ... below row1

    // The producer thread sets the barriers up and starts the weight stream at once; weights never depend on the
    // previous grid, so under programmatic dependent launch this runs while that grid is still computing.
    const bool is_producer = (warp == GEMV_CONSUMER_WARPS);
    int issued = 0;
    int next_row = row0;  // producer: first row not yet requested
    if (is_producer && lane == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        GEMV_TRACE_ANY(8);
        mbar_init_fence();
    }
    for (int i = tid; i < counter_ints; i += GEMV_THREADS) counters[i] = 0;
    __syncthreads();  // barriers initialised: the consumers go on to their activations, the producer to its copies
    GEMV_TRACE(1);
    if (is_producer && lane == 0) {
        GEMV_TRACE_ANY(5);
        int r = row0;
        for (; r < row1 && issued < S; ++issued) {
            const int rows = min(R, row1 - r);
            const uint32_t bytes = ((uint32_t)rows * (uint32_t)p.row_bytes + 15u) & ~15u;
            mbar_arrive_expect_tx(&full[issued], bytes);
            bulk_copy_g2s(ring + (size_t)issued * p.stage_bytes, p.w + (size_t)r * p.row_bytes, bytes, &full[issued]);
            r += rows;
        }
        next_row = r;
        GEMV_TRACE_ANY(9);
        if (r >= row1) prefetch_successor(p.next, cta);  // everything of this CTA is already on its way
    }

    if (is_producer) {
        // ---------------- producer: refills stages as the consumers release them ----------------
        if (lane == 0) {
            bool ok = true;
            int s = 0;          // the refills start over at stage 0 (issued == S here whenever this loop runs)
            uint32_t ph = 0;    // parity of the consumers' first release of each stage
            for (int it = issued, r = next_row; r < row1 && ok; ++it, r += R) {
                ok = mbar_wait_bounded(&empty[s], ph);
                if (!ok) { record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, it); break; }
                const int rows = min(R, row1 - r);
                const uint32_t bytes = ((uint32_t)rows * (uint32_t)p.row_bytes + 15u) & ~15u;
                mbar_arrive_expect_tx(&full[s], bytes);
                bulk_copy_g2s(ring + (size_t)s * p.stage_bytes, p.w + (size_t)r * p.row_bytes, bytes, &full[s]);
                issued = it + 1;
                if (r + R >= row1) prefetch_successor(p.next, cta);
                if (++s == S) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            if (!ok) {
                // a consumer may have left; wait (bounded) until every copy already issued has landed so that no
                // copy writes into shared memory after this CTA is gone
                for (int it = max(0, issued - S); it < issued; ++it) {
                    if (!mbar_wait_bounded(&full[it % S], (it / S) & 1)) {
                        record_failure(p.status, STATUS_WAIT_DRAIN_TIMEOUT, it);
                        break;
                    }
                }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    if (p.use_pdl) {
        grid_dependency_wait();  // the previous grid has finished and its stores are visible
        pre.issue(p.act, B, p.K, p.stride_act, p.act_vec != 0, tid);
    }
#if B200Q_GEMV_TRACE
    if (p.trace != nullptr && tid == 0) {  // when this thread's first activation load has come back
        if constexpr (ACT == ACT_Q8_1) asm volatile("" ::"r"(pre.v[0]));
        else asm volatile("" ::"r"(pre.raw[0][0]));
        GEMV_TRACE(10);
    }
#endif
    if constexpr (ACT == ACT_Q8_1)
        stage_acts_q8_1<B>(acts, reinterpret_cast<const uint8_t*>(p.act), p.K, p.stride_act, tid, GEMV_CONSUMER_THREADS, pre);
    else
        stage_acts_raw<B, act_t, TYPE, ACT>(acts, reinterpret_cast<const act_t*>(p.act), p.K, p.stride_act, p.act_vec != 0, tid,
                                            GEMV_CONSUMER_THREADS, pre);
    GEMV_TRACE(6);
    named_bar_sync(1, GEMV_CONSUMER_THREADS);
    GEMV_TRACE(2);

    const int nrec = p.K / 64;
    const int items = p.K / 128;
    const int islots = 1 << p.log2_islots;  // lanes that share one row inside a warp
    const int rpw = 32 >> p.log2_islots;    // rows a warp works on at once
    const int lane_i = lane & (islots - 1), lane_r = lane >> p.log2_islots;
    const int nrg = GEMV_CONSUMER_WARPS >> p.log2_wpr;  // warp groups working on different rows
    const int wgroup = warp >> p.log2_wpr, wslice = warp & (WPR - 1);
    const int row_slot = wgroup * rpw + lane_r;  // this lane's row within a pass of nrg * rpw rows
    const int rows_per_pass = nrg * rpw;
    const int item0 = wslice * 32 + lane_i;
    const int item_step = 32 * WPR;
    const uint32_t acts_addr = smem_u32(acts);
    const uint32_t ring_addr = smem_u32(ring);
    const uint32_t act_row_bytes = (uint32_t)nrec * ACT_REC_BYTES;
    dst_t* dst = reinterpret_cast<dst_t*>(p.dst);

    Acts<TYPE> areg[NREG > 0 ? B : 1][NREG > 0 ? NREG : 1];
    if (NREG > 0) {
#pragma unroll
        for (int b = 0; b < B; ++b)
#pragma unroll
            for (int j = 0; j < (NREG > 0 ? NREG : 1); ++j)
                if (item0 + j * item_step < items) areg[b][j].load(acts_addr + b * act_row_bytes, item0 + j * item_step);
    }

    // Row-parallel matmul with the exchange fused in (peer_allreduce.cuh): the CTA keeps its rows of the output in shared
    // memory and, when its last row is done, pushes them to every rank and sums what the same CTA of every rank pushed.
    unsigned int ar_epoch = 0;
    dst_t* ar_stage = reinterpret_cast<dst_t*>(smem + p.ar_offset);
    if constexpr (AR) {
        // the call number: one more than the finished launches (published by the last CTA of the previous launch,
        // which this grid was ordered after - by the stream, or by grid_dependency_wait above under programmatic launch)
        ar_epoch = par_next_epoch(*reinterpret_cast<volatile unsigned int*>(par_header(p.px) + PAR_EPOCH_FUSED));
    }
    auto store_out = [&](int b, int row, float v) {
        if constexpr (AR) ar_stage[b * p.ar_rows + (row - row0)] = from_float<dst_t>(v);
        else dst[(size_t)b * p.stride_dst + row] = from_float<dst_t>(v);
    };
    GEMV_TRACE(7);
    bool alive = true;
    // ring position and row rotation kept incrementally: the loop has no integer division
    int s = 0;
    uint32_t ph = 0;
    int rot = 0;
    int rot_step = R;  // R mod rows_per_pass (R is at most a few passes)
    while (rot_step >= rows_per_pass) rot_step -= rows_per_pass;
    for (int it = 0, rbase = row0; rbase < row1; rbase += R, ++it) {
        if (alive && !mbar_wait_bounded(&full[s], ph)) {
            record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, it);
            alive = false;  // keep arriving so that the others are not held up, but compute nothing
        }
        if (it == 0) GEMV_TRACE(3);
        else if (it <= 2) GEMV_TRACE(10 + 2 * it);  // 12, 14: stages 1 and 2 landed
        const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
        const int rows_here = min(R, row1 - rbase);
        // rows of consecutive stages go to consecutive warp groups, so a stage may hold fewer rows than one pass of
        // all warps without leaving the same warps idle every time
        const int my_slot = row_slot >= rot ? row_slot - rot : row_slot - rot + rows_per_pass;
        if constexpr (NREG > 0) {
            // Two rows per warp in flight (rows r and r + rows_per_pass of the stage): their loads, dot products and
            // shuffle reductions are independent, so one row's latencies hide behind the other's work. Everything is
            // computed unconditionally on clamped addresses and masked afterwards, which keeps it one basic block.
            // (With two item slots per lane a row already gives two independent chains, and two rows would spill.)
            constexpr int U = NREG == 1 ? 2 : 1;
            for (int pass0 = 0; pass0 < rows_here; pass0 += U * rows_per_pass) {  // warp-uniform trip count
                int r_in[U];
                bool has_row[U];
                float acc[U][B];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    r_in[u] = pass0 + my_slot + u * rows_per_pass;
                    has_row[u] = r_in[u] < rows_here;
#pragma unroll
                    for (int b = 0; b < B; ++b) acc[u][b] = 0.0f;
                }
#pragma unroll
                for (int j = 0; j < NREG; ++j) {
                    const int item = item0 + j * item_step;
                    const bool item_ok = item < items;
                    const int item_c = item_ok ? item : 0;
                    Weights<TYPE> W[U];
#pragma unroll
                    for (int u = 0; u < U; ++u)
                        W[u].load(st + (uint32_t)(has_row[u] ? r_in[u] : 0) * (uint32_t)p.row_bytes, item_c);
#pragma unroll
                    for (int u = 0; u < U; ++u)
#pragma unroll
                        for (int b = 0; b < B; ++b) {
                            const float d = dot(W[u], areg[b][j]);
                            acc[u][b] += (alive && has_row[u] && item_ok) ? d : 0.0f;
                        }
                }
                // reduce over the lanes that share the row
#pragma unroll
                for (int m = 16; m > 0; m >>= 1) {
                    if (m < islots) {
#pragma unroll
                        for (int u = 0; u < U; ++u)
#pragma unroll
                            for (int b = 0; b < B; ++b) acc[u][b] += __shfl_xor_sync(0xffffffffu, acc[u][b], m);
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (lane_i == 0 && has_row[u]) {
                        if (WPR == 1) {
#pragma unroll
                            for (int b = 0; b < B; ++b) store_out(b, rbase + r_in[u], acc[u][b]);
                        } else {
                            // the last of the WPR warps to arrive adds the partial sums in slice order and writes the row
                            float* part = partial + ((size_t)(s * R + r_in[u]) * WPR) * B;
#pragma unroll
                            for (int b = 0; b < B; ++b) part[wslice * B + b] = acc[u][b];
                            __threadfence_block();
                            const int arrived = atomicAdd(&counters[s * R + r_in[u]], 1);
                            if (arrived == WPR - 1) {
                                __threadfence_block();
                                counters[s * R + r_in[u]] = 0;
#pragma unroll
                                for (int b = 0; b < B; ++b) {
                                    float v = 0.0f;
                                    for (int w = 0; w < WPR; ++w) v += reinterpret_cast<volatile float*>(part)[w * B + b];
                                    store_out(b, rbase + r_in[u], v);
                                }
                            }
                        }
                    }
                }
            }
        } else {
            for (int pass0 = 0; pass0 < rows_here; pass0 += rows_per_pass) {  // warp-uniform trip count
                const int r_in = pass0 + my_slot;
                const bool has_row = r_in < rows_here;
                float acc[B];
#pragma unroll
                for (int b = 0; b < B; ++b) acc[b] = 0.0f;
                if (alive && has_row) {
                    const uint32_t row_addr = st + (uint32_t)r_in * (uint32_t)p.row_bytes;
                    for (int j = 0; j < IPL; ++j) {
                        const int item = item0 + j * item_step;
                        if (item < items) {
                            Weights<TYPE> W;
                            W.load(row_addr, item);
#pragma unroll
                            for (int b = 0; b < B; ++b) {
                                Acts<TYPE> A;
                                A.load(acts_addr + b * act_row_bytes, item);
                                acc[b] += dot(W, A);
                            }
                        }
                    }
                }
                // reduce over the lanes that share the row
#pragma unroll
                for (int m = 16; m > 0; m >>= 1) {
                    if (m < islots) {
#pragma unroll
                        for (int b = 0; b < B; ++b) acc[b] += __shfl_xor_sync(0xffffffffu, acc[b], m);
                    }
                }
                if (lane_i == 0 && has_row) {
                    if (WPR == 1) {
#pragma unroll
                        for (int b = 0; b < B; ++b) store_out(b, rbase + r_in, acc[b]);
                    } else {
                        // the last of the WPR warps to arrive adds the partial sums in slice order and writes the row
                        float* part = partial + ((size_t)(s * R + r_in) * WPR) * B;
#pragma unroll
                        for (int b = 0; b < B; ++b) part[wslice * B + b] = acc[b];
                        __threadfence_block();
                        const int arrived = atomicAdd(&counters[s * R + r_in], 1);
                        if (arrived == WPR - 1) {
                            __threadfence_block();
                            counters[s * R + r_in] = 0;
#pragma unroll
                            for (int b = 0; b < B; ++b) {
                                float v = 0.0f;
                                for (int w = 0; w < WPR; ++w) v += reinterpret_cast<volatile float*>(part)[w * B + b];
                                store_out(b, rbase + r_in, v);
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (it == 0) GEMV_TRACE(11);
        else if (it <= 2) GEMV_TRACE(11 + 2 * it);  // 13, 15: stages 1 and 2 consumed
        if (++s == S) {
            s = 0;
            ph ^= 1u;
        }
        rot += rot_step;
        if (rot >= rows_per_pass) rot -= rows_per_pass;
    }
    if constexpr (AR) exchange_cta_rows<dst_t, B>(p.px, ar_stage, p.ar_rows, row0, row1, p.N, p.dst, p.status, tid, ar_epoch);
    GEMV_TRACE(4);
}

// ---------------------------------------------------------------------------------------------
// Grouped GEMV: up to four weight matrices with the same K applied to the same single activation row in ONE launch
// (q/k/v of an attention block, gate/up of an MLP: the reference's fused_qkv / fused_glu matvecs,
// crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:761-962, without the activation epilogue). The matrices may
// have different types and row counts; each has its own output. The fixed cost of a launch (launch gap, barrier set-up,
// activation quantization, first bytes from HBM) is paid once for the group. Every CTA takes its share of the rows of
// every matrix, one matrix after the other, through the same stage ring.
// ---------------------------------------------------------------------------------------------
constexpr int GEMV_GROUP_MAX = 4;

struct GemvGroupParams {
    const uint8_t* w[GEMV_GROUP_MAX];
    void* dst[GEMV_GROUP_MAX];
    int N[GEMV_GROUP_MAX];
    int type[GEMV_GROUP_MAX];
    int row_bytes[GEMV_GROUP_MAX];
    int rows_per_stage[GEMV_GROUP_MAX];
    int row_align[GEMV_GROUP_MAX];
    int units_per_cta[GEMV_GROUP_MAX];
    int units_extra[GEMV_GROUP_MAX];
    int cta_shift[GEMV_GROUP_MAX];  // matrix m's partition starts at this CTA, so that each matrix's extra units go to other CTAs
    int nmat;
    const void* act;  // one raw activation row of K values
    int K;
    int warps_per_row, items_per_lane, log2_wpr, log2_islots;
    int nstages, stage_bytes, act_bytes, max_rows_per_stage;
    int use_pdl, act_vec;
    unsigned int* status;
    NextPrefetch next;
    PeerExchange px;  // px.world > 1 (one matrix only): the row-parallel matmul with the exchange fused in, as gemv_staged_kernel
    int ar_rows, ar_offset;
};

// rows [row0, row1) of matrix m that CTA `cta` owns
__device__ __forceinline__ void group_rows(const GemvGroupParams& p, int m, int cta, int& row0, int& row1) {
    cta -= p.cta_shift[m];
    if (cta < 0) cta += (int)gridDim.x;
    const int unit0 = cta * p.units_per_cta[m] + min(cta, p.units_extra[m]);
    row0 = unit0 * p.row_align[m];
    row1 = (unit0 + p.units_per_cta[m] + (cta < p.units_extra[m] ? 1 : 0)) * p.row_align[m];
    if (row1 > p.N[m]) row1 = p.N[m];
    if (row1 < row0) row1 = row0;
}

template <int TYPE, typename dst_t, int NREG, bool ONE_ROW_TURNS>
__device__ __forceinline__ void group_stage_rows(const GemvGroupParams& p, uint32_t st, int row_bytes, int rows_here, int rbase,
                                                 int my_slot, int rows_per_pass, int item0, int item_step, int items, int islots,
                                                 int lane_i, int WPR, int wslice, int IPL, uint32_t acts_addr,
                                                 const ActPair (&areg)[NREG > 0 ? NREG : 1], float* part_base, int* cnt_base,
                                                 dst_t* dst, bool alive) {
    if constexpr (NREG > 0) {
        // two rows per warp in flight, computed unconditionally on clamped addresses and masked (see gemv_staged_kernel)
        constexpr int U = NREG == 1 ? 2 : 1;
        // one turn for UU rows per warp: rows pass0 + my_slot + u * rows_per_pass
        auto turn = [&](auto uu_tag, int pass0) {
            constexpr int UU = decltype(uu_tag)::value;
            int r_in[UU];
            bool has_row[UU];
            float acc[UU];
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                r_in[u] = pass0 + my_slot + u * rows_per_pass;
                has_row[u] = r_in[u] < rows_here;
                acc[u] = 0.0f;
            }
#pragma unroll
            for (int j = 0; j < NREG; ++j) {
                const int item = item0 + j * item_step;
                const bool item_ok = item < items;
                const int item_c = item_ok ? item : 0;
                Weights<TYPE> W[UU];
#pragma unroll
                for (int u = 0; u < UU; ++u) W[u].load(st + (uint32_t)(has_row[u] ? r_in[u] : 0) * (uint32_t)row_bytes, item_c);
#pragma unroll
                for (int u = 0; u < UU; ++u) {
                    const float d = dot(W[u], areg[j]);
                    acc[u] += (alive && has_row[u] && item_ok) ? d : 0.0f;
                }
            }
            if (islots == 32) {  // a whole warp per row (every K from 4096 up): no per-level test
#pragma unroll
                for (int m = 16; m > 0; m >>= 1) {
#pragma unroll
                    for (int u = 0; u < UU; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], m);
                }
            } else {
#pragma unroll
                for (int m = 8; m > 0; m >>= 1)
                    if (m < islots) {
#pragma unroll
                        for (int u = 0; u < UU; ++u) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], m);
                    }
            }
#pragma unroll
            for (int u = 0; u < UU; ++u) {
                if (lane_i == 0 && has_row[u]) {
                    if (WPR == 1) {
                        dst[rbase + r_in[u]] = from_float<dst_t>(acc[u]);
                    } else {
                        float* part = part_base + (size_t)r_in[u] * WPR;
                        part[wslice] = acc[u];
                        __threadfence_block();
                        const int arrived = atomicAdd(&cnt_base[r_in[u]], 1);
                        if (arrived == WPR - 1) {
                            __threadfence_block();
                            cnt_base[r_in[u]] = 0;
                            float v = 0.0f;
                            for (int w = 0; w < WPR; ++w) v += reinterpret_cast<volatile float*>(part)[w];
                            dst[rbase + r_in[u]] = from_float<dst_t>(v);
                        }
                    }
                }
            }
        };
        for (int pass0 = 0; pass0 < rows_here; pass0 += U * rows_per_pass) {
            // a warp none of whose lanes has a row in this pass (the short last stage of a CTA's range) leaves the
            // issue slots to the warps that have one. A warp without a second row takes the turn for one row where that
            // saves the most, on Q6_K rows: a second copy of the loop body for every type and in the variant with the
            // fused exchange as well made the tensor-parallel chain, where the two variants alternate, 7 % slower.
            if (!__any_sync(0xffffffffu, pass0 + my_slot < rows_here)) continue;
            if (U == 2 && ONE_ROW_TURNS && TYPE == TYPE_Q6_K && !__any_sync(0xffffffffu, pass0 + my_slot + rows_per_pass < rows_here))
                turn(std::integral_constant<int, 1>{}, pass0);
            else
                turn(std::integral_constant<int, U>{}, pass0);
        }
    } else {
        for (int pass0 = 0; pass0 < rows_here; pass0 += rows_per_pass) {
            const int r_in = pass0 + my_slot;
            const bool has_row = r_in < rows_here;
            float acc = 0.0f;
            if (alive && has_row) {
                const uint32_t row_addr = st + (uint32_t)r_in * (uint32_t)row_bytes;
                for (int j = 0; j < IPL; ++j) {
                    const int item = item0 + j * item_step;
                    if (item < items) {
                        Weights<TYPE> W;
                        W.load(row_addr, item);
                        ActPair A;
                        A.load(acts_addr, item);
                        acc += dot(W, A);
                    }
                }
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1)
                if (m < islots) acc += __shfl_xor_sync(0xffffffffu, acc, m);
            if (lane_i == 0 && has_row) {
                if (WPR == 1) {
                    dst[rbase + r_in] = from_float<dst_t>(acc);
                } else {
                    float* part = part_base + (size_t)r_in * WPR;
                    part[wslice] = acc;
                    __threadfence_block();
                    const int arrived = atomicAdd(&cnt_base[r_in], 1);
                    if (arrived == WPR - 1) {
                        __threadfence_block();
                        cnt_base[r_in] = 0;
                        float v = 0.0f;
                        for (int w = 0; w < WPR; ++w) v += reinterpret_cast<volatile float*>(part)[w];
                        dst[rbase + r_in] = from_float<dst_t>(v);
                    }
                }
            }
        }
    }
}

// ACT: ACT_RAW_Q8_1 (raw row, quantized here to Q8_1 as the two-launch protocol does) or ACT_Q8_1 (blocks already
// quantized by the caller: the reference's fused q/k/v launcher)
template <typename dst_t, typename act_t, int NREG, int ACT = ACT_RAW_Q8_1, bool AR = false>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_group_kernel(const GemvGroupParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GEMV_MAX_STAGES;
    uint8_t* acts = smem + GEMV_BARRIER_BYTES;
    const int S = p.nstages, WPR = p.warps_per_row, IPL = p.items_per_lane, RMAX = p.max_rows_per_stage;
    float* partial = reinterpret_cast<float*>(acts + p.act_bytes);  // [S][RMAX][WPR]
    const int partial_floats = WPR > 1 ? S * RMAX * WPR : 0;
    int* counters = reinterpret_cast<int*>(partial + partial_floats);  // [S][RMAX]
    const int counter_ints = WPR > 1 ? S * RMAX : 0;
    uint8_t* ring = acts + p.act_bytes + (((partial_floats + counter_ints) * 4 + 127) & ~127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    // programmatic dependent launch: as in gemv_staged_kernel, only the consumers wait for the previous grid, and only
    // after the CTA-wide barrier, so that the producer starts the weight stream at once
    if (p.use_pdl) grid_launch_dependents();
    ActPrefetch<ACT, act_t> pre;
    if (!p.use_pdl && warp != GEMV_CONSUMER_WARPS) pre.issue(p.act, 1, p.K, p.K, p.act_vec != 0, tid);

    const bool is_producer = (warp == GEMV_CONSUMER_WARPS);
    if (is_producer && lane == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        mbar_init_fence();
    }
    for (int i = tid; i < counter_ints; i += GEMV_THREADS) counters[i] = 0;
    __syncthreads();

    if (is_producer) {
        // ---------------- producer: this CTA's rows of every matrix, in order, through one ring ----------------
        if (lane == 0) {
            bool ok = true;
            int g = 0;  // running stage number over all matrices
            int s = 0;
            uint32_t ph = 1;  // becomes the parity of the consumers' first release once the ring has gone round
            for (int m = 0; m < p.nmat && ok; ++m) {
                int row0, row1;
                group_rows(p, m, cta, row0, row1);
                const int R = p.rows_per_stage[m];
                for (int r = row0; r < row1 && ok; r += R, ++g) {
                    if (g >= S) {
                        ok = mbar_wait_bounded(&empty[s], ph);
                        if (!ok) { record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, g); break; }
                    }
                    const int rows = min(R, row1 - r);
                    const uint32_t bytes = ((uint32_t)rows * (uint32_t)p.row_bytes[m] + 15u) & ~15u;
                    mbar_arrive_expect_tx(&full[s], bytes);
                    bulk_copy_g2s(ring + (size_t)s * p.stage_bytes, p.w[m] + (size_t)r * p.row_bytes[m], bytes, &full[s]);
                    if (++s == S) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            if (ok) prefetch_successor(p.next, cta);
            if (!ok) {
                for (int q = max(0, g - S); q < g; ++q)
                    if (!mbar_wait_bounded(&full[q % S], (q / S) & 1)) {
                        record_failure(p.status, STATUS_WAIT_DRAIN_TIMEOUT, q);
                        break;
                    }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    if (p.use_pdl) {
        grid_dependency_wait();
        pre.issue(p.act, 1, p.K, p.K, p.act_vec != 0, tid);
    }
    // the activation row is quantized once for all matrices
    if constexpr (ACT == ACT_Q8_1) {
        stage_acts_q8_1<1>(acts, reinterpret_cast<const uint8_t*>(p.act), p.K, 0, tid, GEMV_CONSUMER_THREADS, pre);
    } else if constexpr (ACT == ACT_RAW_CPU) {
        // the CPU path's format depends on the weight type (Q8_K for the K-quants, Q8_0 for Q8_0): the launcher admits
        // only groups whose matrices agree on it
        if (p.type[0] == TYPE_Q8_0)
            stage_acts_raw<1, act_t, TYPE_Q8_0, ACT>(acts, reinterpret_cast<const act_t*>(p.act), p.K, p.K, p.act_vec != 0, tid,
                                                     GEMV_CONSUMER_THREADS, pre);
        else
            stage_acts_raw<1, act_t, TYPE_Q4_K, ACT>(acts, reinterpret_cast<const act_t*>(p.act), p.K, p.K, p.act_vec != 0, tid,
                                                     GEMV_CONSUMER_THREADS, pre);
    } else {
        stage_acts_raw<1, act_t, TYPE_Q4_K, ACT>(acts, reinterpret_cast<const act_t*>(p.act), p.K, p.K, p.act_vec != 0, tid,
                                                 GEMV_CONSUMER_THREADS, pre);
    }
    named_bar_sync(1, GEMV_CONSUMER_THREADS);

    const int items = p.K / 128;
    const int islots = 1 << p.log2_islots;
    const int rpw = 32 >> p.log2_islots;
    const int lane_i = lane & (islots - 1), lane_r = lane >> p.log2_islots;
    const int nrg = GEMV_CONSUMER_WARPS >> p.log2_wpr;
    const int wgroup = warp >> p.log2_wpr, wslice = warp & (WPR - 1);
    const int row_slot = wgroup * rpw + lane_r;
    const int rows_per_pass = nrg * rpw;
    const int item0 = wslice * 32 + lane_i;
    const int item_step = 32 * WPR;
    const uint32_t acts_addr = smem_u32(acts);
    const uint32_t ring_addr = smem_u32(ring);

    ActPair areg[NREG > 0 ? NREG : 1];
    if (NREG > 0) {
#pragma unroll
        for (int j = 0; j < (NREG > 0 ? NREG : 1); ++j)
            if (item0 + j * item_step < items) areg[j].load(acts_addr, item0 + j * item_step);
    }

    // fused exchange (one matrix): the CTA's outputs go to shared memory first, then to every rank
    unsigned int ar_epoch = 0;
    dst_t* ar_stage = reinterpret_cast<dst_t*>(smem + p.ar_offset);
    if constexpr (AR) ar_epoch = par_next_epoch(*reinterpret_cast<volatile unsigned int*>(par_header(p.px) + PAR_EPOCH_FUSED));

    bool alive = true;
    int g = 0;
    int s = 0;
    uint32_t ph = 0;
    int rot = 0;  // rows handed out so far modulo rows_per_pass: rotates the row-to-warp assignment across stages
    for (int m = 0; m < p.nmat; ++m) {
        int row0, row1;
        group_rows(p, m, cta, row0, row1);
        const int R = p.rows_per_stage[m];
        const int mtype = p.type[m];
        dst_t* dst = AR ? ar_stage - row0 : reinterpret_cast<dst_t*>(p.dst[m]);
        for (int r = row0; r < row1; r += R, ++g) {
            if (alive && !mbar_wait_bounded(&full[s], ph)) {
                record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, g);
                alive = false;
            }
            const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
            const int rows_here = min(R, row1 - r);
            // (rows_per_pass is a power of two: both the warp groups and the rows per warp are)
            const int my_slot = (row_slot - rot) & (rows_per_pass - 1);
            rot = (rot + rows_here) & (rows_per_pass - 1);
            float* part_base = partial + (size_t)s * RMAX * WPR;
            int* cnt_base = counters + s * RMAX;
            if (mtype == TYPE_Q4_K)
                group_stage_rows<TYPE_Q4_K, dst_t, NREG, !AR>(p, st, p.row_bytes[m], rows_here, r, my_slot, rows_per_pass, item0, item_step,
                                                         items, islots, lane_i, WPR, wslice, IPL, acts_addr, areg, part_base, cnt_base, dst, alive);
            else if (mtype == TYPE_Q6_K)
                group_stage_rows<TYPE_Q6_K, dst_t, NREG, !AR>(p, st, p.row_bytes[m], rows_here, r, my_slot, rows_per_pass, item0, item_step,
                                                         items, islots, lane_i, WPR, wslice, IPL, acts_addr, areg, part_base, cnt_base, dst, alive);
            else
                group_stage_rows<TYPE_Q8_0, dst_t, NREG, !AR>(p, st, p.row_bytes[m], rows_here, r, my_slot, rows_per_pass, item0, item_step,
                                                         items, islots, lane_i, WPR, wslice, IPL, acts_addr, areg, part_base, cnt_base, dst, alive);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (++s == S) {
                s = 0;
                ph ^= 1u;
            }
        }
    }
    if constexpr (AR) {
        int row0, row1;
        group_rows(p, 0, cta, row0, row1);
        exchange_cta_rows<dst_t, 1>(p.px, ar_stage, p.ar_rows, row0, row1, p.N[0], p.dst[0], p.status, tid, ar_epoch);
    }
}

// ---------------------------------------------------------------------------------------------
// Simple kernel: one warp per weight row, byte-granular loads, Q8_1 activations read from global memory. Used when
// the staged kernel's preconditions do not hold (unaligned weights, activations too large for shared memory).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int ld_i8(const uint8_t* p) { return (int)(int8_t)*p; }

template <int TYPE, int B, typename dst_t>
__global__ void __launch_bounds__(256) gemv_simple_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ vy,
                                                          dst_t* __restrict__ dst, int K, int N, int stride_act,
                                                          int stride_dst, int use_pdl) {
    if (use_pdl) grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= N) return;
    const int nb32 = K / 32;
    const size_t row_bytes = (size_t)(K / type_block_elems(TYPE)) * type_block_bytes(TYPE);
    const uint8_t* rp = w + (size_t)row * row_bytes;
    float acc[B];
#pragma unroll
    for (int b = 0; b < B; ++b) acc[b] = 0.0f;
    for (int kb = lane; kb < nb32; kb += 32) {  // one 32-value group per lane
        int wq[32];
        float scale = 0.0f, minv = 0.0f;
        if (TYPE == TYPE_Q8_0) {
            const uint8_t* blk = rp + (size_t)kb * Q8_0_BYTES;
            scale = half_bits_to_float((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
            for (int l = 0; l < 32; ++l) wq[l] = ld_i8(blk + 2 + l);
        } else if (TYPE == TYPE_Q4_K) {
            const int s = kb >> 3, j = kb & 7;
            const uint8_t* sb = rp + (size_t)s * Q4_K_BYTES;
            const uint8_t* q = sb + 4;
            int sc, m;
            if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
            else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
            scale = half_bits_to_float((uint32_t)sb[0] | ((uint32_t)sb[1] << 8)) * (float)sc;
            minv = half_bits_to_float((uint32_t)sb[2] | ((uint32_t)sb[3] << 8)) * (float)m;
            const uint8_t* qs = sb + 16 + 32 * (j >> 1);
            for (int l = 0; l < 32; ++l) wq[l] = (j & 1) ? (qs[l] >> 4) : (qs[l] & 0xF);
        } else {
            const int s = kb >> 3, n = (kb >> 2) & 1, qd = kb & 3;
            const uint8_t* sb = rp + (size_t)s * Q6_K_BYTES;
            const uint8_t* ql = sb + 64 * n + 32 * (qd & 1);
            const uint8_t* qh = sb + 128 + 32 * n;
            for (int l = 0; l < 32; ++l) {
                const int lo = (qd & 2) ? (ql[l] >> 4) : (ql[l] & 0xF);
                const int hi = (qh[l] >> (2 * qd)) & 3;
                wq[l] = (lo | (hi << 4)) - 32;
            }
            scale = half_bits_to_float((uint32_t)sb[208] | ((uint32_t)sb[209] << 8));
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const uint8_t* ab = vy + ((size_t)b * stride_act + kb) * Q8_1_BYTES;
            const float d8 = half_bits_to_float((uint32_t)ab[0] | ((uint32_t)ab[1] << 8));
            if (TYPE == TYPE_Q6_K) {
                const int s = kb >> 3, n = (kb >> 2) & 1, qd = kb & 3;
                const uint8_t* sb = rp + (size_t)s * Q6_K_BYTES;
                int d0 = 0, d1 = 0;
                for (int l = 0; l < 16; ++l) d0 += wq[l] * ld_i8(ab + 4 + l);
                for (int l = 16; l < 32; ++l) d1 += wq[l] * ld_i8(ab + 4 + l);
                const float s0 = (float)ld_i8(sb + 192 + 8 * n + 2 * qd), s1 = (float)ld_i8(sb + 192 + 8 * n + 2 * qd + 1);
                acc[b] += scale * d8 * (s0 * (float)d0 + s1 * (float)d1);
            } else {
                int dotv = 0, s8 = 0;
                for (int l = 0; l < 32; ++l) {
                    const int a = ld_i8(ab + 4 + l);
                    dotv += wq[l] * a;
                    s8 += a;
                }
                acc[b] += scale * d8 * (float)dotv - minv * d8 * (float)s8;
            }
        }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const float v = warp_sum(acc[b]);
        if (lane == 0) dst[(size_t)b * stride_dst + row] = from_float<dst_t>(v);
    }
}

// ---------------------------------------------------------------------------------------------
// Host-side planning and dispatch
// ---------------------------------------------------------------------------------------------
static inline int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

struct GemvPlan {
    bool staged;
    GemvParams p;
    int grid;
    int nreg;  // register-resident item slots per lane (0 = activations read from shared memory)
    size_t smem;
};

// Chooses the lane-to-item mapping, rows per stage, ring depth and grid for a shape. `w` is only inspected for
// alignment (nullptr = assume aligned).
static inline GemvPlan plan_gemv(int type, int K, int N, int B, const void* w, int out_piece_rows = 1) {
    const RuntimeInfo& rt = runtime_info();
    GemvPlan plan{};
    GemvParams& p = plan.p;
    const int be = type_block_elems(type), bb = type_block_bytes(type);
    p.K = K;
    p.N = N;
    p.row_bytes = K / be * bb;
    p.row_align = 16 / gcd_int(p.row_bytes, 16);
    // fused exchange (out_piece_rows > 1): every CTA's row range is whole 8-byte pieces of the output, and the CTA keeps
    // its outputs in shared memory until it exchanges them
    if (out_piece_rows > 1) p.row_align = p.row_align * out_piece_rows / gcd_int(p.row_align, out_piece_rows);
    long long units = (N + p.row_align - 1) / p.row_align;
    long long grid = rt.sm_count;
    if (grid > units) grid = units;
    if (grid < 1) grid = 1;
    p.ar_rows = (int)((units + grid - 1) / grid) * p.row_align;
    const int ar_bytes = out_piece_rows > 1 ? ((B * p.ar_rows * 4 + 127) & ~127) : 0;
    p.act_bytes = ((B * (K / 64) * ACT_REC_BYTES) + 127) & ~127;
    p.use_pdl = rt.use_pdl;
    plan.staged = false;
    if (rt.force_simple || K % 128 != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0) return plan;

    const int items = K / 128;
    int islots = 32;
    while (islots > 1 && (islots >> 1) >= items) islots >>= 1;
    const int rpw = 32 / islots;
    // a row of more than 32 items: up to 2 item slots per lane (their activations stay in registers for one
    // activation row), then more warps per row
    int ipl = 1, wpr = 1;
    if (items > 32) {
        const int regs_ipl = (B == 1) ? 2 : 1;
        while (wpr * 32 * ipl < items) {
            if (ipl < regs_ipl) ipl *= 2;
            else if (wpr < GEMV_CONSUMER_WARPS) wpr *= 2;
            else ipl *= 2;
        }
        // prefer one slot per lane when that does not need more warps than two slots would
        if (ipl == 2 && wpr * 32 >= items) ipl = 1;
    }
    // keep a stage (one pass of all warps) under ~48 KB: trade the second slot for more warps per row
    while (ipl > 1 && wpr < GEMV_CONSUMER_WARPS &&
           (long long)(GEMV_CONSUMER_WARPS / wpr) * rpw * p.row_bytes > rt.gemv_pass_limit) {
        ipl /= 2;
        wpr *= 2;
    }
    if (ipl > 16) return plan;
    const int nrg = GEMV_CONSUMER_WARPS / wpr;
    const int rows_per_pass = nrg * rpw;
    // rows per stage: whole passes of all warps (every warp visits every stage in order, so a stage that feeds only
    // some warps would stall the others), about gemv_stage_target bytes, at least one pass
    // register-resident activations: 40 registers per slot and activation row
    plan.nreg = (B == 1 && ipl <= 2) ? ipl : ((B == 2 && ipl == 1) ? 1 : 0);
    // with one register-resident slot a warp keeps two rows of a stage in flight (rows r and r + rows_per_pass), so a
    // stage holds two passes
    const int passes = plan.nreg == 1 ? (rt.gemv_passes == 1 ? 1 : 2) : 1;
    const int unit = rows_per_pass * p.row_align / gcd_int(rows_per_pass, p.row_align) * passes;
    int R = passes * rt.gemv_stage_target / (unit * p.row_bytes) * unit;
    if (R < unit) R = unit;
    p.rows_per_stage = R;
    p.warps_per_row = wpr;
    p.items_per_lane = ipl;
    p.log2_wpr = 0;
    while ((1 << p.log2_wpr) < wpr) ++p.log2_wpr;
    p.log2_islots = 0;
    while ((1 << p.log2_islots) < islots) ++p.log2_islots;
    p.stage_bytes = (R * p.row_bytes + 16 + 127) & ~127;
    const int budget = rt.smem_optin - 1024 - ar_bytes;  // one CTA per SM; 1 KB per CTA is reserved by the system
    int S = 0;
    for (;;) {
        p.rows_per_stage = R;
        p.stage_bytes = (R * p.row_bytes + 16 + 127) & ~127;
        for (S = GEMV_MAX_STAGES; S >= 2; --S) {
            const int combine = wpr > 1 ? (((S * R * wpr * B + S * R) * 4 + 127) & ~127) : 0;
            if (GEMV_BARRIER_BYTES + p.act_bytes + combine + S * p.stage_bytes <= budget) {
                plan.smem = (size_t)GEMV_BARRIER_BYTES + p.act_bytes + combine + (size_t)S * p.stage_bytes;
                break;
            }
        }
        // large batches leave little room beside their activations: hold fewer rows than one pass of all warps
        if (S >= 2 || R <= p.row_align || (R / 2) % p.row_align != 0) break;
        R /= 2;
    }
    if (S < 2) return plan;  // does not fit: simple kernel
    p.nstages = S;
    R = p.rows_per_stage;
    // A CTA with several stages of rows gets them in whole stages: a ragged last stage costs a CTA a full turn of the
    // stage loop for a few rows (twice in a grouped launch of two such matrices), which is more than the extra stage
    // that some CTAs then have over the others.
    // Only where few CTAs end up with the extra stage (they then draw more than their share of HBM): with 3 or 4 stages
    // each for half of the CTAs (Q6_K 14336 x 4096) it is slower. And only for short launches: over the 27 stages per CTA
    // of an output head the ragged stage is amortised, and a dozen CTAs left alone with a 100 KB stage cost 2 us.
    if (out_piece_rows == 1 && (long long)N / R >= 2 * grid) {
        const long long stages = ((long long)N + R - 1) / R;
        if (stages % grid <= grid / 4 && stages / grid < 8) {
            p.row_align = R;
            units = stages;
        }
    }
    p.ar_offset = (int)plan.smem;
    plan.smem += ar_bytes;
    plan.grid = (int)grid;
    p.units_per_cta = (int)(units / grid);
    p.units_extra = (int)(units % grid);
    plan.staged = true;
    return plan;
}

// The successor registered for weight matrix `w`, cut as its own launch will cut it (see NextPrefetch).
static inline NextPrefetch plan_next_prefetch(const void* w);

template <typename Kern>
static inline cudaError_t launch_gemv_kernel(Kern kernel, int grid, int block, size_t smem, cudaStream_t s, bool pdl,
                                             const GemvParams& p) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3((unsigned)block, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, p);
}

static inline NextPrefetch plan_next_prefetch(const void* w) {
    NextPrefetch n{};
    const RuntimeInfo& rt = runtime_info();
    WeightSuccessor succ;
    const int prefetch_bytes = l2_prefetch_bytes_effective(rt);
    if (prefetch_bytes < 16 || !find_weight_successor(w, &succ)) return n;
    if (type_block_bytes(succ.type) == 0 || succ.K <= 0 || succ.N <= 0 || succ.K % type_block_elems(succ.type) != 0) return n;
    const GemvPlan next = plan_gemv(succ.type, succ.K, succ.N, 1, succ.w);
    if (!next.staged) return n;
    n.w = static_cast<const uint8_t*>(succ.w);
    n.total_bytes = ((long long)succ.N * next.p.row_bytes) & ~15LL;
    n.unit_bytes = next.p.row_align * next.p.row_bytes;
    n.units_per_cta = next.p.units_per_cta;
    n.units_extra = next.p.units_extra;
    n.grid = next.grid;
    n.bytes = prefetch_bytes & ~15;
    return n;
}

template <int TYPE, int B, typename dst_t, int ACT, typename act_t, int NREG, bool AR>
static inline int launch_staged_ar(const GemvPlan& plan, cudaStream_t s) {
    auto kernel = gemv_staged_kernel<TYPE, B, dst_t, ACT, act_t, NREG, AR>;
    static PerDeviceOnce configured;  // per instantiation
    cudaError_t e = configured.run([&] {
        return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, runtime_info().smem_optin - 1024);
    });
    if (e != cudaSuccess) return (int)e;
    return (int)launch_gemv_kernel(kernel, plan.grid, GEMV_THREADS, plan.smem, s, plan.p.use_pdl != 0, plan.p);
}

template <int TYPE, int B, typename dst_t, int ACT, typename act_t, int NREG>
static inline int launch_staged_n(const GemvPlan& plan, cudaStream_t s) {
    if (plan.p.px.world > 1) {
        // the fused exchange exists for raw activations in the decode quantizer's arithmetic (what b200q_gemv runs)
        if constexpr (ACT == ACT_RAW_Q8_1) return launch_staged_ar<TYPE, B, dst_t, ACT, act_t, NREG, true>(plan, s);
        else return B200Q_ERR_UNSUPPORTED;
    }
    return launch_staged_ar<TYPE, B, dst_t, ACT, act_t, NREG, false>(plan, s);
}

template <int TYPE, int B, typename dst_t, int ACT, typename act_t>
static inline int launch_staged(const GemvPlan& plan, cudaStream_t s) {
    if (B == 1 && plan.nreg == 2) return launch_staged_n<TYPE, B, dst_t, ACT, act_t, (B == 1 ? 2 : 0)>(plan, s);
    if (B <= 2 && plan.nreg == 1) return launch_staged_n<TYPE, B, dst_t, ACT, act_t, (B <= 2 ? 1 : 0)>(plan, s);
    return launch_staged_n<TYPE, B, dst_t, ACT, act_t, 0>(plan, s);
}

// (defined once, in gemv_group.cu: every caller must reach the SAME copy of the grouped kernel)
int gemv_group(int elem, int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, const void* x,
               cudaStream_t s, const PeerExchange* px, int act_mode);

template <int TYPE, int B, typename dst_t>
static inline int launch_gemv_b(const void* vx, const void* act, void* dst, int K, int N, int stride_act, int stride_dst,
                                int act_mode, const PeerExchange* px, cudaStream_t s) {
    const bool exchange = px != nullptr && px->world > 1;
    if (B == 1 && (act_mode == ACT_RAW_Q8_1 || (act_mode == ACT_RAW_CPU && !exchange)) && runtime_info().gemv_one_kernel) {
        // One row of raw activations: the grouped kernel with a single matrix - the same arithmetic in the same order, a
        // little more bookkeeping per row, but a decode chain then alternates between fewer kernels, and its launches
        // are sensitive to how much code they have to fetch (+2 % on the chain).
        const int type = TYPE;
        constexpr int elem = sizeof(dst_t) == 4 ? ELEM_F32 : (std::is_same<dst_t, __half>::value ? ELEM_F16 : ELEM_BF16);
        if (!exchange || stride_dst == N) {
            const int rc = gemv_group(elem, 1, &type, &vx, &dst, &N, K, act, s, exchange ? px : nullptr, act_mode);
            if (rc != B200Q_ERR_UNSUPPORTED) return rc;
        }
    }
    constexpr int PIECE = 8 / (int)sizeof(dst_t);  // output rows per 8-byte piece of the exchange
    if (exchange) {
        // fused all-reduce: contiguous [B][N] output, rows of whole 8-byte pieces, within the capacity; staged kernel only
        const long long bytes = (long long)B * N * (long long)sizeof(dst_t);
        if (stride_dst != N || N % PIECE != 0 || bytes > px->capacity || reinterpret_cast<uintptr_t>(dst) % 8 != 0) return B200Q_ERR_UNSUPPORTED;
    }
    GemvPlan plan = plan_gemv(TYPE, K, N, B, vx, exchange ? PIECE : 1);
    if (exchange && !plan.staged) return B200Q_ERR_UNSUPPORTED;
    plan.p.w = (const uint8_t*)vx;
    plan.p.act = act;
    plan.p.dst = dst;
    plan.p.stride_act = stride_act;
    plan.p.stride_dst = stride_dst;
    plan.p.status = status_ptr();
    plan.p.trace = trace_slot();
    plan.p.px.world = 0;
    if (exchange) plan.p.px = *px;
    plan.p.next = plan_next_prefetch(vx);
    if (plan.staged) {
        if (act_mode == ACT_Q8_1) return launch_staged<TYPE, B, dst_t, ACT_Q8_1, float>(plan, s);
        // raw activations have the output's type
        plan.p.act_vec = (reinterpret_cast<uintptr_t>(act) % 16 == 0) && ((size_t)stride_act * sizeof(dst_t) % 16 == 0);
        if (act_mode == ACT_RAW_CPU && TYPE != TYPE_Q8_0 && K % 256 != 0) return B200Q_ERR_UNSUPPORTED;
        if (act_mode == ACT_RAW_CPU) return launch_staged<TYPE, B, dst_t, ACT_RAW_CPU, dst_t>(plan, s);
        return launch_staged<TYPE, B, dst_t, ACT_RAW_Q8_1, dst_t>(plan, s);
    }
    if (act_mode != ACT_Q8_1) return B200Q_ERR_UNSUPPORTED;  // the simple kernel needs Q8_1 blocks
    gemv_simple_kernel<TYPE, B, dst_t><<<(N + 7) / 8, 256, 0, s>>>((const uint8_t*)vx, (const uint8_t*)act, (dst_t*)dst, K, N,
                                                                 stride_act, stride_dst, 0);
    return (int)cudaGetLastError();
}

template <int TYPE, typename dst_t>
static inline int launch_gemv(const void* vx, const void* act, void* dst, int K, int N, int stride_act, int stride_dst,
                              int b, int act_mode, const PeerExchange* px, cudaStream_t s) {
    if (N <= 0 || K <= 0) return 0;
    switch (b) {
        case 1: return launch_gemv_b<TYPE, 1, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        case 2: return launch_gemv_b<TYPE, 2, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        case 3: return launch_gemv_b<TYPE, 3, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        case 4: return launch_gemv_b<TYPE, 4, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        case 5: return launch_gemv_b<TYPE, 5, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        case 6: return launch_gemv_b<TYPE, 6, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        case 7: return launch_gemv_b<TYPE, 7, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        case 8: return launch_gemv_b<TYPE, 8, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, px, s);
        default: return B200Q_ERR_UNSUPPORTED;
    }
}

// Plans and launches a grouped GEMV (one activation row). Returns B200Q_ERR_UNSUPPORTED when the group does not fit
// the staged kernel's preconditions; the caller then launches the matrices one by one.
template <typename dst_t, int ACT = ACT_RAW_Q8_1>
static inline int launch_gemv_group(int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K,
                                    const void* x, cudaStream_t s, const PeerExchange* px = nullptr) {
    const RuntimeInfo& rt = runtime_info();
    if (nmat < 1 || nmat > GEMV_GROUP_MAX || K <= 0 || K % 128 != 0 || rt.force_simple) return B200Q_ERR_UNSUPPORTED;
    // fused exchange: one matrix, rows of whole 8-byte pieces, within the capacity (as launch_gemv_b checks it)
    const bool exchange = px != nullptr && px->world > 1;
    constexpr int PIECE = 8 / (int)sizeof(dst_t);
    if (exchange && (nmat != 1 || ACT != ACT_RAW_Q8_1 || Ns[0] % PIECE != 0 || (long long)Ns[0] * (long long)sizeof(dst_t) > px->capacity ||
                     reinterpret_cast<uintptr_t>(dsts[0]) % 8 != 0))
        return B200Q_ERR_UNSUPPORTED;
    if (ACT == ACT_RAW_CPU) {
        // one activation format for the whole group: all Q8_0 (blocks of 32) or all K-quants (superblocks of 256)
        for (int m = 0; m < nmat; ++m)
            if ((types[m] == TYPE_Q8_0) != (types[0] == TYPE_Q8_0)) return B200Q_ERR_UNSUPPORTED;
        if (types[0] != TYPE_Q8_0 && K % 256 != 0) return B200Q_ERR_UNSUPPORTED;
    }
    GemvGroupParams p{};
    p.nmat = nmat;
    p.K = K;
    p.act = x;
    p.act_bytes = (((K / 64) * ACT_REC_BYTES) + 127) & ~127;
    p.act_vec = (reinterpret_cast<uintptr_t>(x) % 16 == 0);
    p.use_pdl = rt.use_pdl;
    p.status = status_ptr();
    p.next = plan_next_prefetch(ws[nmat - 1]);
    int grid = rt.sm_count, max_stage = 0, max_R = 0, wpr = 0, ipl = 0;
    for (int m = 0; m < nmat; ++m) {
        if (type_block_bytes(types[m]) == 0 || K % type_block_elems(types[m]) != 0) return B200Q_ERR_UNSUPPORTED;
        if (reinterpret_cast<uintptr_t>(ws[m]) % 16 != 0 || Ns[m] <= 0) return B200Q_ERR_UNSUPPORTED;
        const GemvPlan one = plan_gemv(types[m], K, Ns[m], 1, ws[m], exchange ? PIECE : 1);
        if (!one.staged) return B200Q_ERR_UNSUPPORTED;
        p.ar_rows = one.p.ar_rows;
        if (m == 0) { wpr = one.p.warps_per_row; ipl = one.p.items_per_lane; p.log2_wpr = one.p.log2_wpr; p.log2_islots = one.p.log2_islots; }
        if (one.p.warps_per_row != wpr || one.p.items_per_lane != ipl) return B200Q_ERR_UNSUPPORTED;  // same K: cannot differ
        p.w[m] = static_cast<const uint8_t*>(ws[m]);
        p.dst[m] = dsts[m];
        p.N[m] = Ns[m];
        p.type[m] = types[m];
        p.row_bytes[m] = one.p.row_bytes;
        p.rows_per_stage[m] = one.p.rows_per_stage;
        p.row_align[m] = one.p.row_align;
        if (one.p.stage_bytes > max_stage) max_stage = one.p.stage_bytes;
        if (one.p.rows_per_stage > max_R) max_R = one.p.rows_per_stage;
    }
    int shift = 0;
    for (int m = 0; m < nmat; ++m) {
        const long long units = (p.N[m] + p.row_align[m] - 1) / p.row_align[m];
        p.units_per_cta[m] = (int)(units / grid);
        p.units_extra[m] = (int)(units % grid);
        p.cta_shift[m] = exchange ? 0 : shift;  // (the first matrix stays in place: the L2 prefetch of a successor assumes it)
        shift = (shift + p.units_extra[m]) % grid;
    }
    p.warps_per_row = wpr;
    p.items_per_lane = ipl;
    p.stage_bytes = max_stage;
    p.max_rows_per_stage = max_R;
    const int ar_bytes = exchange ? ((p.ar_rows * 4 + 127) & ~127) : 0;
    const int budget = rt.smem_optin - 1024 - ar_bytes;
    int S = 0;
    size_t smem = 0;
    for (S = GEMV_MAX_STAGES; S >= 2; --S) {
        const int combine = wpr > 1 ? (((S * max_R * wpr + S * max_R) * 4 + 127) & ~127) : 0;
        if (GEMV_BARRIER_BYTES + p.act_bytes + combine + S * max_stage <= budget) {
            smem = (size_t)GEMV_BARRIER_BYTES + p.act_bytes + combine + (size_t)S * max_stage;
            break;
        }
    }
    if (S < 2) return B200Q_ERR_UNSUPPORTED;
    p.nstages = S;
    p.ar_offset = (int)smem;
    smem += ar_bytes;
    if (exchange) p.px = *px;
    const int nreg = ipl <= 2 ? ipl : 0;
    auto launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, rt.smem_optin - 1024);
        if (e != cudaSuccess) return (int)e;
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)grid, 1, 1);
        cfg.blockDim = dim3(GEMV_THREADS, 1, 1);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = p.use_pdl ? 1 : 0;
        return (int)cudaLaunchKernelEx(&cfg, kernel, p);
    };
    using act_t = typename std::conditional<ACT == ACT_Q8_1, float, dst_t>::type;
    if constexpr (ACT == ACT_RAW_Q8_1) {
        if (exchange) {
            if (nreg == 1) return launch(gemv_group_kernel<dst_t, act_t, 1, ACT, true>);
            if (nreg == 2) return launch(gemv_group_kernel<dst_t, act_t, 2, ACT, true>);
            return launch(gemv_group_kernel<dst_t, act_t, 0, ACT, true>);
        }
    }
    if (nreg == 1) return launch(gemv_group_kernel<dst_t, act_t, 1, ACT>);
    if (nreg == 2) return launch(gemv_group_kernel<dst_t, act_t, 2, ACT>);
    return launch(gemv_group_kernel<dst_t, act_t, 0, ACT>);
}

// One weight type's dispatcher over the output element type; defined once per type in gemv_<type>.cu.
template <int TYPE>
static inline int gemv_type_dispatch(int dst_elem, const void* vx, const void* act, void* dst, int K, int N, int stride_act,
                                     int stride_dst, int b, int act_mode, const PeerExchange* px, cudaStream_t s) {
    if (dst_elem == ELEM_BF16) return launch_gemv<TYPE, __nv_bfloat16>(vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, px, s);
    if (dst_elem == ELEM_F16) return launch_gemv<TYPE, __half>(vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, px, s);
    if (dst_elem == ELEM_F32) return launch_gemv<TYPE, float>(vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, px, s);
    return B200Q_ERR_UNSUPPORTED;
}

}  // namespace b200q

// The reference's launcher symbols for one type (crates/inference-quant/src/gguf/ffi.rs:846-878); stride_col_y is in
// Q8_1 blocks. Launchers return nothing, as the reference's: a failed launch surfaces at the caller's next checked
// CUDA call, and is also kept for b200q_take_launch_status().
#define B200Q_DEFINE_GEMV_TYPE(tag, TYPE)                                                                              \
    namespace b200q {                                                                                                  \
    int gemv_##tag(int dst_elem, const void* vx, const void* act, void* dst, int K, int N, int stride_act,             \
                   int stride_dst, int b, int act_mode, const PeerExchange* px, cudaStream_t s) {                      \
        return note_launch_status(                                                                                     \
            gemv_type_dispatch<TYPE>(dst_elem, vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, px, s));       \
    }                                                                                                                  \
    }                                                                                                                  \
    extern "C" void launch_mmvq_gguf_##tag##_bf16_plain(const void* vx, const void* vy, void* dst, int ncols_x,        \
                                                        int nrows_x, int stride_col_y, int stride_col_dst, int b_size, \
                                                        void* stream) {                                                \
        b200q::gemv_##tag(b200q::ELEM_BF16, vx, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst, b_size,       \
                          b200q::ACT_Q8_1, nullptr, (cudaStream_t)stream);                                                      \
    }                                                                                                                  \
    extern "C" void launch_mmvq_gguf_##tag##_f16_plain(const void* vx, const void* vy, void* dst, int ncols_x,         \
                                                       int nrows_x, int stride_col_y, int stride_col_dst, int b_size,  \
                                                       void* stream) {                                                 \
        b200q::gemv_##tag(b200q::ELEM_F16, vx, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst, b_size,        \
                          b200q::ACT_Q8_1, nullptr, (cudaStream_t)stream);                                                      \
    }                                                                                                                  \
    extern "C" void launch_mmvq_gguf_##tag##_f32_plain(const void* vx, const void* vy, void* dst, int ncols_x,         \
                                                       int nrows_x, int stride_col_y, int stride_col_dst, int b_size,  \
                                                       void* stream) {                                                 \
        b200q::gemv_##tag(b200q::ELEM_F32, vx, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst, b_size,        \
                          b200q::ACT_Q8_1, nullptr, (cudaStream_t)stream);                                                      \
    }

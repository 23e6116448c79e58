// Small batches (1..16 activation rows) on the tcgen05 tensor cores with 8-bit integer operands: every packed weight
// block is read from HBM once and decoded once for all rows. Takes the place of the reference's tensor-core matvec
// tier: host side fast_mmvq::tiled_plain (crates/inference-quant/src/gguf/fast_mmvq.rs:2049-2126), activation layout
// kernel mmvq_tc_quantize (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_quantize.cu:157-190), matvec
// mmvq_tc_k_kernel (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_tc_k.cuh:221-329). Same arithmetic as there:
// activations become int8 with one scale per 32 values (d = amax / 127 stored as f16, q = roundf(x / d), integer block
// sums for the min term), the 32-value dot products are exact integers, and scales are applied in f32.
//
// Two launches:
//   1. tcq_quantize_kernel: x [M][K] -> int8 matrix q [16][K] (rows >= M zero) plus float2 (d, d * sum q) per
//      (32-value block, row). For Q6_K, whose scales cover 16 values, q has 32 rows: rows 0..15 keep only the first
//      half of every 32-value block and rows 16..31 only the second, so that one 32-deep MMA yields both halves'
//      sums in separate accumulator columns.
//   2. gemv_tc_i8_kernel: one persistent CTA per SM owns a contiguous run of weight rows and walks it in tiles of up
//      to 128 rows (= TMEM lanes). Per stage of 256 k:
//        warp 3       TMA (2-D tensor map over the packed bytes) brings the tile's 256-k chunk of every row;
//        warps 4-11   (two groups of four on alternate stages) unpack quants to int8 into a K-major
//                     128-byte-swizzled A stage, and the rows' block scales to f32 into a side buffer;
//        warp 0       TMA brings the activation tile (B operand) and its scales;
//        warp 1       issues 8 tcgen05.mma kind::i8 (M = 128, N = 16 or 32, K = 32), one per 32-value block, each
//                     into its own TMEM columns (no accumulation across blocks: scales differ);
//        warps 12-27  read the integer sums from TMEM (thread = weight row), apply block and activation scales and
//                     accumulate in f32 registers; at the end of a tile they store the outputs.
//      TMEM holds several stages' sums so that scaling stage g overlaps the MMAs of the following stages.
//      A matrix with too few rows to give every SM a useful tile (N <= 74 tiles of 128 rows) is split along K as
//      well: each CTA takes a run of 256-k stages of ONE full-height tile, writes its partial outputs to the
//      workspace, and the last CTA to arrive for a tile's 32-row quarter adds the partials in split order.
//
// Every wait is bounded; a wait that gives up records a code in the device status word, work is skipped, and the
// kernel still frees its TMEM columns before it returns.
#include "common.cuh"
#include "runtime.h"
#include "tcgen05.cuh"

namespace b200q {

constexpr int TCQ_TOKENS = 16;
constexpr int TCQ_ROWS = 128;                  // tile rows = TMEM lanes
constexpr int TCQ_KC = 256;                    // k per stage
constexpr int TCQ_SC_STAGES = 3;
constexpr int TCQ_SC_PITCH = 80;               // bytes per row of block scales: 16 floats + padding against bank conflicts
constexpr int TCQ_SC_BYTES = TCQ_ROWS * TCQ_SC_PITCH;
constexpr int TCQ_DS_BYTES = 8 * TCQ_TOKENS * 8;  // activation scales of a stage: float2 [8 blocks][16 rows]
constexpr int TCQ_UNPACK_WARPS = 8;            // warps 4..11
constexpr int TCQ_SCALE_WARPS = 16;            // warps 12..27
constexpr int TCQ_THREADS = 32 * (4 + TCQ_UNPACK_WARPS + TCQ_SCALE_WARPS);
constexpr int TCQ_OUT_BYTES = TCQ_ROWS * TCQ_TOKENS * 4;  // partial-sum exchange between the scaling warps of a row
constexpr int TCQ_SMEM_LIMIT = 232448;
constexpr int TCQ_MAX_CTAS = 160;                       // K-split mode: at most one CTA per SM
constexpr int TCQ_COUNTERS = TCQ_MAX_CTAS * 4;          // one per (tile, TMEM lane quarter)
constexpr size_t TCQ_PARTIAL_BYTES = (size_t)TCQ_MAX_CTAS * TCQ_ROWS * TCQ_TOKENS * sizeof(float);  // sum over tiles of ksplit * 16 * rows

// X_STAGES: the activation ring is deep because an SM's loads return in order: a tile requested now arrives after the
// packed-row stages already in flight, several stage times later.
template <int TYPE> struct TcqType;
template <> struct TcqType<TYPE_Q4_K> { static constexpr int CHUNK = 144, PITCH = 144, XROWS = 16, X_STAGES = 8; };
template <> struct TcqType<TYPE_Q6_K> { static constexpr int CHUNK = 210, PITCH = 240, XROWS = 32, X_STAGES = 6; };
template <> struct TcqType<TYPE_Q8_0> { static constexpr int CHUNK = 272, PITCH = 272, XROWS = 16, X_STAGES = 8; };

template <int TYPE> struct TcqLayout {
    using TT = TcqType<TYPE>;
    static constexpr int X_BYTES = TT::XROWS * TCQ_KC + TCQ_DS_BYTES;  // two sub-tiles of XROWS x 128 bytes, then the scales
    // everything but the A and packed-row rings: alignment slack, activation ring, block scales, exchange buffer, barriers
    static constexpr int FIXED = 1024 + TT::X_STAGES * X_BYTES + TCQ_SC_STAGES * TCQ_SC_BYTES + TCQ_OUT_BYTES + 512;
    static constexpr int NCOL = TT::XROWS;             // accumulator columns per 32-value block
    static constexpr int BUF_COLS = 8 * NCOL;          // per stage
    static constexpr int TMEM_BUFS = 512 / BUF_COLS;   // stages of sums held at once: 4 or 2
    static constexpr int TMEM_COLS = 512;
};

struct TcqBarriers {
    uint64_t raw_full[8], raw_empty[8];
    uint64_t a_full[4], a_empty[4];
    uint64_t sc_full[TCQ_SC_STAGES], sc_empty[TCQ_SC_STAGES];
    uint64_t x_full[8], x_empty[8];
    uint64_t tmem_full[4], tmem_empty[4];
    uint64_t comb[4];  // end of a tile: comb[i] = the warps of block pair i have added their sums (3: read them)
    uint32_t tmem_base;
};
static_assert(sizeof(TcqBarriers) <= 512, "barrier block");

struct TcqParams {
    void* y;            // [M][ldy]
    const uint8_t* ds;  // float2 [K / 32][16]
    int M, N, K, ldy;
    int tile_rows;                 // rows a tile loads (multiple of 8, <= 128)
    int a_stages, raw_stages;      // ring depths (2..4 and 2..8), as many as the tile's stage sizes leave room for
    int rows_per_cta, rows_extra;  // CTA c owns rows [c * q + min(c, r), ...) with q = rows_per_cta, r = rows_extra
    // matrices with too few rows to give every SM a useful tile are split along K as well: ksplit > 1 makes CTA c take
    // the 256-k stages [s * nkc / ksplit, (s + 1) * nkc / ksplit), s = c % ksplit, of the single tile c / ksplit; the
    // splits' partial outputs meet in `partial` [ksplit][16][N] and the last to arrive (counter per tile and lane
    // quarter, zeroed by the quantize launch) adds them in split order and stores
    int ksplit;
    float* partial;
    unsigned int* counters;
    unsigned int* status;
    unsigned long long* trace;  // optional: SM clock of CTA 0's pipeline events, [event 0..7][stage 0..trace_stages)
    int trace_stages;
    // REF_ACTS kernels: the activations as the reference's mmvq_tc_quantize lays them out (tcq_ref_quantize_kernel
    // below writes the same bytes): `ref_halves` halves of 8 rows, each K / 32 blocks of 288 bytes
    const uint8_t* ref_acts;
    int ref_halves;
};

#define TCQ_TRACE(event, g)                                                                          \
    do {                                                                                             \
        if (p.trace != nullptr && blockIdx.x == 0 && (g) < p.trace_stages)                           \
            p.trace[(event) * p.trace_stages + (g)] = (unsigned long long)clock64();                 \
    } while (0)

// ---------------------------------------------------------------------------------------------
// Launch 1: activations -> int8 rows + per-block scales. One CTA per 32-value block, one warp per activation row.
// ---------------------------------------------------------------------------------------------
template <typename src_t, bool SPLIT_HALVES>
__global__ void __launch_bounds__(32 * TCQ_TOKENS) tcq_quantize_kernel(const src_t* __restrict__ x, int8_t* __restrict__ q,
                                                                      float2* __restrict__ ds, int K, int M, int ldx,
                                                                      unsigned int* __restrict__ counters) {
    const int kb = blockIdx.x, row = threadIdx.y, lane = threadIdx.x;
    // the matvec launch that follows may start now: until its own dependency wait it only sets up and streams weights
    grid_launch_dependents();
    if (kb == 0) {  // the K-split arrival counters of the launch that follows
        const int i = row * 32 + lane;
        for (int c = i; c < TCQ_COUNTERS; c += 32 * TCQ_TOKENS) counters[c] = 0u;
    }
    const int k = kb * 32 + lane;
    const float xi = row < M ? to_float<src_t>(x[(size_t)row * ldx + k]) : 0.0f;
    const float amax = warp_max(fabsf(xi));
    const float d = amax / 127.0f;
    const int qi = amax == 0.0f ? 0 : (int)roundf(xi / d);
    const int sum = __reduce_add_sync(0xffffffffu, qi);
    if (SPLIT_HALVES) {
        q[(size_t)row * K + k] = (int8_t)(lane < 16 ? qi : 0);
        q[(size_t)(TCQ_TOKENS + row) * K + k] = (int8_t)(lane < 16 ? 0 : qi);
    } else {
        q[(size_t)row * K + k] = (int8_t)qi;
    }
    if (lane == 0) {
        const float dh = __half2float(__float2half_rn(d));
        ds[(size_t)kb * TCQ_TOKENS + row] = make_float2(dh, dh * (float)sum);
    }
}

// The reference tier's own activation layout (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_quantize.cu:148-190,
// mmvq_tc_act.cuh:1-7), for hosts that call launch_mmvq_tc_quantize_* / launch_mmvq_tc_gguf_*_plain as a pair: the
// rows in halves of 8, one half after the other; per half nb = gridDim.x blocks of 32 values: nb * 32 int2 (entry
// 4r + t of a block = row r's values 4t..4t+3 then 16+4t..16+4t+3), then nb * 8 f16 scales d = amax / 127, then nb * 8
// int16 sums of the quants q = roundf(x / d). One CTA per (block, half), one warp per row.
constexpr int TCQ_REF_BLOCK_BYTES = 32 * 8 + 8 * 2 + 8 * 2;  // 288
template <typename src_t>
__global__ void __launch_bounds__(256) tcq_ref_quantize_kernel(const src_t* __restrict__ x, uint8_t* __restrict__ vy, int kx, int num_rows) {
    const int ib = blockIdx.x, nb = gridDim.x, row = threadIdx.y, lane = threadIdx.x;
    const int col = ib * 32 + lane;
    const int input_row = blockIdx.y * 8 + row;
    uint8_t* base = vy + (size_t)blockIdx.y * nb * TCQ_REF_BLOCK_BYTES;
    const float xi = (input_row < num_rows && col < kx) ? to_float<src_t>(x[(size_t)input_row * kx + col]) : 0.0f;
    const float amax = warp_max(fabsf(xi));
    const float d = amax / 127.0f;
    const int qi = amax == 0.0f ? 0 : (int)roundf(xi / d);
    const int sum = __reduce_add_sync(0xffffffffu, qi);
    __shared__ __align__(8) int8_t q[8][32];
    q[row][lane] = (int8_t)qi;
    if (lane == 0) {
        reinterpret_cast<__half*>(base + (size_t)nb * 256)[ib * 8 + row] = __float2half_rn(d);
        reinterpret_cast<int16_t*>(base + (size_t)nb * 256 + (size_t)nb * 16)[ib * 8 + row] = (int16_t)sum;
    }
    __syncthreads();
    if (row == 0) {
        const int r = lane >> 2, t = lane & 3;
        reinterpret_cast<int2*>(base)[(size_t)ib * 32 + lane] =
            make_int2(*reinterpret_cast<const int*>(&q[r][4 * t]), *reinterpret_cast<const int*>(&q[r][16 + 4 * t]));
    }
}

__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) { asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory"); }

// One stage (256 k = 8 blocks) of the reference-layout activations -> the B-operand tile the MMAs read (XROWS rows of
// 128 swizzled bytes per 128-k sub-tile; for Q6_K rows 0..15 carry the first 16 values of every block and rows 16..31
// the last 16) plus float2 (d, d * sum) per (block, row). Rows the caller did not supply stay zero. By one warp.
template <int TYPE>
__device__ __forceinline__ void tcq_stage_ref_acts(const TcqParams& p, int kc, uint8_t* st, int lane) {
    using TT = TcqType<TYPE>;
    using L = TcqLayout<TYPE>;
    const uint32_t st_addr = smem_u32(st);
    for (int i = lane; i < L::X_BYTES / 16; i += 32) sts128(st_addr + 16 * i, 0u, 0u, 0u, 0u);
    __syncwarp();
    const int nb = p.K / 32;
    const int r = lane >> 2, t = lane & 3;
    for (int hf = 0; hf < p.ref_halves; ++hf) {
        const uint8_t* base = p.ref_acts + (size_t)hf * nb * TCQ_REF_BLOCK_BYTES;
        const int row = hf * 8 + r;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int2 frag = __ldg(reinterpret_cast<const int2*>(base) + (size_t)(8 * kc + j) * 32 + lane);
            const uint32_t sub = st_addr + (uint32_t)(j >> 2) * (TT::XROWS * 128);
            const int c = 2 * (j & 3);
            if constexpr (TYPE == TYPE_Q6_K) {
                sts32(b_chunk_addr(sub, row, c) + 4 * t, (uint32_t)frag.x);
                sts32(b_chunk_addr(sub, TCQ_TOKENS + row, c + 1) + 4 * t, (uint32_t)frag.y);
            } else {
                sts32(b_chunk_addr(sub, row, c) + 4 * t, (uint32_t)frag.x);
                sts32(b_chunk_addr(sub, row, c + 1) + 4 * t, (uint32_t)frag.y);
            }
        }
        // scales and sums of the stage's 8 blocks x 8 rows: two entries per lane
        const __half* ds = reinterpret_cast<const __half*>(base + (size_t)nb * 256);
        const int16_t* ss = reinterpret_cast<const int16_t*>(base + (size_t)nb * 256 + (size_t)nb * 16);
#pragma unroll
        for (int e2 = 0; e2 < 2; ++e2) {
            const int e = lane + 32 * e2, j = e >> 3, rr = e & 7;
            const float dh = __half2float(ds[(8 * kc + j) * 8 + rr]);
            const float sm = (float)(int)ss[(8 * kc + j) * 8 + rr];
            float2* dst = reinterpret_cast<float2*>(st + TT::XROWS * TCQ_KC) + j * TCQ_TOKENS + hf * 8 + rr;
            *dst = make_float2(dh, dh * sm);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Unpacking: thread (row r, sub-tile J) turns 128 k of its row into int8 (eight 16-byte units of the A stage) and
// writes that half's block scales. `rb` = shared address of the row's chunk, `a_sub` = of the sub-tile, `sc` = of
// the row's scale record.
// ---------------------------------------------------------------------------------------------
template <int TYPE> struct TcqUnpack;

// Q4_K: 144-byte superblock {f16 d, f16 dmin, 12 bytes of 6-bit scales / mins, 128 bytes of nibbles}; value =
// d * sc_j * q - dmin * m_j (crates/inference-tensor/src/quantized/k_quants.rs:2096-2123). Scale record:
// d * sc_j for j = 0..7, then dmin * m_j.
template <> struct TcqUnpack<TYPE_Q4_K> {
    static __device__ __forceinline__ void run(uint32_t rb, int, int J, int r, uint32_t a_sub, uint32_t sc) {
        const uint4 hdr = lds128(rb);
#pragma unroll
        for (int e = 0; e < 2; ++e) {  // 64 k: low nibbles are sub-block 4J + 2e, high nibbles 4J + 2e + 1
            const uint4 w0 = lds128(rb + 16 + 64 * J + 32 * e), w1 = lds128(rb + 32 + 64 * J + 32 * e);
            const uint32_t m = 0x0f0f0f0fu;
            sts128(b_chunk_addr(a_sub, r, 4 * e + 0), w0.x & m, w0.y & m, w0.z & m, w0.w & m);
            sts128(b_chunk_addr(a_sub, r, 4 * e + 1), w1.x & m, w1.y & m, w1.z & m, w1.w & m);
            sts128(b_chunk_addr(a_sub, r, 4 * e + 2), (w0.x >> 4) & m, (w0.y >> 4) & m, (w0.z >> 4) & m, (w0.w >> 4) & m);
            sts128(b_chunk_addr(a_sub, r, 4 * e + 3), (w1.x >> 4) & m, (w1.y >> 4) & m, (w1.z >> 4) & m, (w1.w >> 4) & m);
        }
        const float d = half_bits_to_float(hdr.x), dmin = half_bits_to_float(hdr.x >> 16);
        float ds[4], ms[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            uint32_t s6, m6;
            if (J == 0) {
                s6 = (hdr.y >> (8 * jj)) & 0x3fu;
                m6 = (hdr.z >> (8 * jj)) & 0x3fu;
            } else {
                const uint32_t lo = (hdr.w >> (8 * jj)) & 0xffu;
                s6 = (lo & 0xfu) | ((((hdr.y >> (8 * jj)) & 0xffu) >> 6) << 4);
                m6 = (lo >> 4) | ((((hdr.z >> (8 * jj)) & 0xffu) >> 6) << 4);
            }
            ds[jj] = d * (float)s6;
            ms[jj] = dmin * (float)m6;
        }
        sts128(sc + 16 * J, __float_as_uint(ds[0]), __float_as_uint(ds[1]), __float_as_uint(ds[2]), __float_as_uint(ds[3]));
        sts128(sc + 32 + 16 * J, __float_as_uint(ms[0]), __float_as_uint(ms[1]), __float_as_uint(ms[2]), __float_as_uint(ms[3]));
    }
};

// Q8_0: eight 34-byte blocks {f16 d, 32 int8} per 256 k; value = d * q. Scale record: d of blocks 0..7.
template <> struct TcqUnpack<TYPE_Q8_0> {
    template <int OFF>
    static __device__ __forceinline__ float block(uint32_t rb, int r, uint32_t a_sub, int unit) {
        constexpr int A = OFF & ~15, O = OFF & 15;
        uint32_t c[12], w[9];
        lds_chunks<3>(rb + A, c);
        extract_words<O, 9>(c, w);  // bytes OFF .. OFF + 35: d, then the quants from byte 2
        uint32_t q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = __funnelshift_r(w[i], w[i + 1], 16);
        sts128(b_chunk_addr(a_sub, r, unit), q[0], q[1], q[2], q[3]);
        sts128(b_chunk_addr(a_sub, r, unit + 1), q[4], q[5], q[6], q[7]);
        return half_bits_to_float(w[0]);
    }
    static __device__ __forceinline__ void run(uint32_t rb, int, int J, int r, uint32_t a_sub, uint32_t sc) {
        float d[4];
        if (J == 0) {
            d[0] = block<0>(rb, r, a_sub, 0);
            d[1] = block<34>(rb, r, a_sub, 2);
            d[2] = block<68>(rb, r, a_sub, 4);
            d[3] = block<102>(rb, r, a_sub, 6);
        } else {
            d[0] = block<136>(rb, r, a_sub, 0);
            d[1] = block<170>(rb, r, a_sub, 2);
            d[2] = block<204>(rb, r, a_sub, 4);
            d[3] = block<238>(rb, r, a_sub, 6);
        }
        sts128(sc + 16 * J, __float_as_uint(d[0]), __float_as_uint(d[1]), __float_as_uint(d[2]), __float_as_uint(d[3]));
    }
};

// Q6_K: 210-byte superblock {ql[128], qh[64], int8 scales[16], f16 d}; value = d * sc_s * (q - 32) with 16 values per
// scale (crates/inference-tensor/src/quantized/k_quants.rs:2649-2680). Half n = J covers k = 128 n + 32 qd + l:
// ql[64 n + 32 (qd & 1) + l] nibble qd >> 1, qh[32 n + l] bits 2 qd. The A operand holds 4 (q - 32) (the six bits
// shifted to the top of the byte, sign bit flipped); the scale record holds d * sc_s / 4 for s = 0..15.
// The chunk starts O = 2 (kc & 7) bytes into its 16-byte-aligned slot (210 kc mod 16).
template <> struct TcqUnpack<TYPE_Q6_K> {
    template <int O>
    static __device__ __forceinline__ void unit(uint32_t rb, int n, int r, uint32_t a_sub, uint32_t sc) {
        uint32_t cl[20], ch[12], ql[16], qh[8];
        lds_chunks<5>(rb + 64 * n, cl);
        lds_chunks<3>(rb + 128 + 32 * n, ch);
        extract_words<O, 16>(cl, ql);
        extract_words<O, 8>(ch, qh);
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            uint32_t v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t l = ql[8 * (qd & 1) + i];
                const uint32_t lo = ((qd >> 1) ? (l >> 2) : (l << 2)) & 0x3c3c3c3cu;
                const uint32_t hi = (qh[i] << (6 - 2 * qd)) & 0xc0c0c0c0u;
                v[i] = (lo | hi) ^ 0x80808080u;
            }
            sts128(b_chunk_addr(a_sub, r, 2 * qd), v[0], v[1], v[2], v[3]);
            sts128(b_chunk_addr(a_sub, r, 2 * qd + 1), v[4], v[5], v[6], v[7]);
        }
        const float d4 = half_bits_to_float(lds16(rb + O + 208)) * 0.25f;
        float s[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t two = lds16(rb + O + 192 + 8 * n + 2 * i);
            s[2 * i] = d4 * (float)(int)(int8_t)(two & 0xffu);
            s[2 * i + 1] = d4 * (float)(int)(int8_t)(two >> 8);
        }
        sts128(sc + 32 * n, __float_as_uint(s[0]), __float_as_uint(s[1]), __float_as_uint(s[2]), __float_as_uint(s[3]));
        sts128(sc + 32 * n + 16, __float_as_uint(s[4]), __float_as_uint(s[5]), __float_as_uint(s[6]), __float_as_uint(s[7]));
    }
    static __device__ __forceinline__ void run(uint32_t rb, int kc, int J, int r, uint32_t a_sub, uint32_t sc) {
        switch (kc & 7) {
            case 0: unit<0>(rb, J, r, a_sub, sc); break;
            case 1: unit<2>(rb, J, r, a_sub, sc); break;
            case 2: unit<4>(rb, J, r, a_sub, sc); break;
            case 3: unit<6>(rb, J, r, a_sub, sc); break;
            case 4: unit<8>(rb, J, r, a_sub, sc); break;
            case 5: unit<10>(rb, J, r, a_sub, sc); break;
            case 6: unit<12>(rb, J, r, a_sub, sc); break;
            default: unit<14>(rb, J, r, a_sub, sc); break;
        }
    }
};

// ---------------------------------------------------------------------------------------------
// TMEM -> registers: TOK consecutive 32-bit columns of this warp's 32 lanes (no wait)
// ---------------------------------------------------------------------------------------------
template <int TOK> __device__ __forceinline__ void tcq_tmem_ld(uint32_t taddr, uint32_t (&r)[TOK]);
template <> __device__ __forceinline__ void tcq_tmem_ld<4>(uint32_t taddr, uint32_t (&r)[4]) { tmem_ld_32x4_nowait(taddr, r); }
template <> __device__ __forceinline__ void tcq_tmem_ld<8>(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
template <> __device__ __forceinline__ void tcq_tmem_ld<16>(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// Scaling of one 32-value block's integer sums for TOK activation rows. `I` (and `Io` for Q6_K's second half) are the
// sums of this thread's weight row; s0 / s1 its block scales (Q4_K: d * sc, dmin * m; Q8_0: d; Q6_K: the two
// halves' d * sc / 4); `dsa` the shared address of float2 (d, d * sum) of the activation rows.
template <int TYPE, int TOK>
__device__ __forceinline__ void tcq_scale_block(const uint32_t (&I)[TOK], const uint32_t (&Io)[TOK], float s0, float s1, uint32_t dsa,
                                                float (&acc)[TOK]) {
#pragma unroll
    for (int t2 = 0; t2 < TOK / 2; ++t2) {
        const uint4 pr = lds128(dsa + 16 * t2);  // rows 2 t2, 2 t2 + 1
        const float xd[2] = {__uint_as_float(pr.x), __uint_as_float(pr.z)};
        const float xs[2] = {__uint_as_float(pr.y), __uint_as_float(pr.w)};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int t = 2 * t2 + u;
            if constexpr (TYPE == TYPE_Q4_K) {
                acc[t] = fmaf(s0, xd[u] * (float)(int)I[t], acc[t]);
                acc[t] = fmaf(-s1, xs[u], acc[t]);
            } else if constexpr (TYPE == TYPE_Q8_0) {
                acc[t] = fmaf(s0, xd[u] * (float)(int)I[t], acc[t]);
            } else {
                acc[t] = fmaf(xd[u], fmaf(s0, (float)(int)I[t], s1 * (float)(int)Io[t]), acc[t]);
            }
        }
    }
}

// Position in a ring of `n` stages: consumers wait for full[i] with parity ph, producers for empty[i] with ph ^ 1.
struct TcqRing {
    int i = 0;
    uint32_t ph = 0;
    __device__ __forceinline__ void next(int n) {
        if (++i == n) {
            i = 0;
            ph ^= 1u;
        }
    }
};

// REF_ACTS: activations come in the reference tier's layout (p.ref_acts) and warp 0 re-lays them out per stage instead
// of fetching ready tiles by TMA.
template <int TYPE, typename dst_t, int TOK, bool REF_ACTS = false>
__global__ void __launch_bounds__(TCQ_THREADS, 1)
    gemv_tc_i8_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x, const TcqParams p) {
    using TT = TcqType<TYPE>;
    using L = TcqLayout<TYPE>;
    constexpr int XS = TT::X_STAGES, TB = L::TMEM_BUFS;
    const int TH = p.tile_rows, NA = p.a_stages, NR = p.raw_stages;
    const int sub_bytes = TH * 128;              // one 128-k sub-tile of the tile's rows; the MMA reads 128 rows, the ones
    const int a_bytes = 2 * sub_bytes;           // beyond the tile from whatever follows in shared memory (never used)
    const int raw_bytes = (TH * TT::PITCH + 127) & ~127;
    extern __shared__ uint8_t tcq_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tcq_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* a_stages = smem;                                                             // [NA][a_bytes]
    uint8_t* x_stages = a_stages + NA * a_bytes;                                          // [XS][X_BYTES], 1024-aligned each
    uint8_t* sc_stages = x_stages + XS * L::X_BYTES;                                      // [3][128 * 80]
    float* out_buf = reinterpret_cast<float*>(sc_stages + TCQ_SC_STAGES * TCQ_SC_BYTES);  // [128][16]
    TcqBarriers* bars = reinterpret_cast<TcqBarriers*>(reinterpret_cast<uint8_t*>(out_buf) + TCQ_OUT_BYTES);
    uint8_t* raw_stages = reinterpret_cast<uint8_t*>(bars) + 512;                         // [NR][raw_bytes]

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = blockIdx.x;
    const int nkc_all = p.K / TCQ_KC;
    int row0, row1, kc0, kc1;
    if (p.ksplit > 1) {
        const int tile = cta / p.ksplit, split = cta - tile * p.ksplit;
        row0 = tile * TH;
        row1 = min(p.N, row0 + TH);
        kc0 = split * nkc_all / p.ksplit;
        kc1 = (split + 1) * nkc_all / p.ksplit;
    } else {
        row0 = cta * p.rows_per_cta + min(cta, p.rows_extra);
        row1 = min(p.N, row0 + p.rows_per_cta + (cta < p.rows_extra ? 1 : 0));
        kc0 = 0;
        kc1 = nkc_all;
    }
    const int ntiles = row1 > row0 ? (row1 - row0 + TH - 1) / TH : 0;
    const int nstages = ntiles * (kc1 - kc0);

    if (tid == 0) {
        for (int s = 0; s < NR; ++s) {
            mbar_init(&bars->raw_full[s], 1);
            mbar_init(&bars->raw_empty[s], TCQ_UNPACK_WARPS / 2);
        }
        for (int s = 0; s < NA; ++s) {
            mbar_init(&bars->a_full[s], TCQ_UNPACK_WARPS / 2);
            mbar_init(&bars->a_empty[s], 1);
        }
        for (int s = 0; s < TCQ_SC_STAGES; ++s) {
            mbar_init(&bars->sc_full[s], TCQ_UNPACK_WARPS / 2);
            mbar_init(&bars->sc_empty[s], TCQ_SCALE_WARPS);
        }
        for (int s = 0; s < XS; ++s) {
            mbar_init(&bars->x_full[s], 1);
            mbar_init(&bars->x_empty[s], TCQ_SCALE_WARPS);
        }
        for (int s = 0; s < TB; ++s) {
            mbar_init(&bars->tmem_full[s], 1);
            mbar_init(&bars->tmem_empty[s], TCQ_SCALE_WARPS);
        }
        for (int s = 0; s < 4; ++s) mbar_init(&bars->comb[s], TCQ_SCALE_WARPS / 4);
        mbar_init_fence();
    }
    if (warp == 2) tmem_alloc(&bars->tmem_base, L::TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    // Launched as a programmatic dependent of the quantize launch (launch_gemv_tc_i8_tok's `after_quantizer`), the CTA
    // got this far, and its packed-row warp streams weights, while the quantizer still runs; what the quantizer writes
    // (activation tiles, scales, the K-split counters) is first touched behind this wait, directly by warp 0 and by
    // every other warp only after a stage that warp 0 has handed on. Without that launch attribute the wait returns at once.
    if (warp == 0) grid_dependency_wait();
    if (warp == 0 && REF_ACTS) {
        // ---------------- activation tiles re-laid out from the reference tier's fragments, by the whole warp ----------------
        TcqRing xr;
        int kc = kc0;
        for (int g = 0; g < nstages; ++g) {
            bool ok = mbar_wait_bounded(&bars->x_empty[xr.i], xr.ph ^ 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, g);
                break;
            }
            tcq_stage_ref_acts<TYPE>(p, kc, x_stages + (size_t)xr.i * L::X_BYTES, lane);
            fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->x_full[xr.i]);
            xr.next(XS);
            if (++kc == kc1) kc = kc0;
        }
    } else if (warp == 0) {
        // ---------------- activation tiles (two XROWS x 128-byte boxes) and their scales ----------------
        if (lane == 0) {
            TcqRing xr;
            int kc = kc0, g = 0;
            bool ok = true;
            for (; g < nstages; ++g) {
                if (!mbar_wait_bounded(&bars->x_empty[xr.i], xr.ph ^ 1)) {
                    record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, g);
                    ok = false;
                    break;
                }
                TCQ_TRACE(0, g);
                uint8_t* st = x_stages + (size_t)xr.i * L::X_BYTES;
                mbar_arrive_expect_tx(&bars->x_full[xr.i], L::X_BYTES);
                tma_load_2d(st, &tmap_x, kc * TCQ_KC, 0, &bars->x_full[xr.i]);
                tma_load_2d(st + TT::XROWS * 128, &tmap_x, kc * TCQ_KC + 128, 0, &bars->x_full[xr.i]);
                bulk_copy_g2s(st + TT::XROWS * TCQ_KC, p.ds + (size_t)kc * TCQ_DS_BYTES, TCQ_DS_BYTES, &bars->x_full[xr.i]);
                xr.next(XS);
                if (++kc == kc1) kc = kc0;
            }
            if (!ok) {  // let the copies already issued land before the CTA may exit: the last min(g, XS) stages
                for (int q = 0; q < min(g, XS); ++q) {
                    // step back one stage
                    if (xr.i == 0) { xr.i = XS - 1; xr.ph ^= 1u; } else --xr.i;
                    if (!mbar_wait_bounded(&bars->x_full[xr.i], xr.ph)) {
                        record_failure(p.status, STATUS_WAIT_DRAIN_TIMEOUT, q);
                        break;
                    }
                }
            }
        }
    } else if (warp == 3) {
        // ---------------- packed rows: one box of tile_rows x chunk bytes per stage ----------------
        if (lane == 0) {
            TcqRing rr;
            int kc = kc0, t = 0, g = 0;
            bool ok = true;
            for (; g < nstages; ++g) {
                if (!mbar_wait_bounded(&bars->raw_empty[rr.i], rr.ph ^ 1)) {
                    record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, 1000 + g);
                    ok = false;
                    break;
                }
                TCQ_TRACE(1, g);
                mbar_arrive_expect_tx(&bars->raw_full[rr.i], (uint32_t)TH * TT::PITCH);
                int xcoord;
                if constexpr (TYPE == TYPE_Q8_0) xcoord = kc * (TT::CHUNK / 2);   // 16-bit elements
                else xcoord = (kc * TT::CHUNK) & ~15;                             // bytes, rounded down to the TMA grain
                tma_load_2d(raw_stages + (size_t)rr.i * raw_bytes, &tmap_w, xcoord, row0 + t * TH, &bars->raw_full[rr.i]);
                rr.next(NR);
                if (++kc == kc1) {
                    kc = kc0;
                    ++t;
                }
            }
            if (!ok) {
                for (int q = 0; q < min(g, NR); ++q) {
                    if (rr.i == 0) { rr.i = NR - 1; rr.ph ^= 1u; } else --rr.i;
                    if (!mbar_wait_bounded(&bars->raw_full[rr.i], rr.ph)) {
                        record_failure(p.status, STATUS_WAIT_DRAIN_TIMEOUT, 1000 + q);
                        break;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: eight independent 128 x NCOL x 32 products per stage ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_i8(1, 1, TCQ_ROWS, L::NCOL);
            // descriptors differ between stages, sub-tiles and 32-byte k steps only in the address field (units of 16 bytes)
            const uint64_t da0 = make_smem_desc_sw128(smem_u32(a_stages));
            const uint64_t dx0 = make_smem_desc_sw128(smem_u32(x_stages));
            const uint32_t sub16 = (uint32_t)sub_bytes >> 4;
            TcqRing ar, xr, tr;
            bool ready = false;  // whether the polls made during the previous stage's issue already found this stage complete
            for (int g = 0; g < nstages; ++g) {
                if (!ready && !mbar_wait3_bounded(&bars->tmem_empty[tr.i], tr.ph ^ 1, &bars->a_full[ar.i], ar.ph, &bars->x_full[xr.i], xr.ph)) {
                    record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, g);
                    break;
                }
                tc_fence_after();
                TCQ_TRACE(4, g);
                const uint64_t da = da0 + (uint64_t)((uint32_t)ar.i * 2u * sub16);
                const uint64_t dx = dx0 + (uint64_t)(xr.i * (L::X_BYTES >> 4));
                const uint32_t d0 = tmem_base + tr.i * L::BUF_COLS;
                const int as = ar.i, ts = tr.i;
                ar.next(NA);
                xr.next(XS);
                tr.next(TB);
                // poll the next stage's barriers now: the answers come back while the MMAs below are being issued (an
                // MMA issue takes about as long as a barrier poll's round trip through the busy shared-memory pipe)
                bool n0 = false, n1 = false, n2 = false;
                if (g + 1 < nstages) {
                    n0 = mbar_try_wait(&bars->tmem_empty[tr.i], tr.ph ^ 1);
                    n1 = mbar_try_wait(&bars->a_full[ar.i], ar.ph);
                    n2 = mbar_try_wait(&bars->x_full[xr.i], xr.ph);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    tc_mma_i8(d0 + j * L::NCOL, da + ((j >> 2) * sub16 + 2 * (j & 3)), dx + ((j >> 2) * ((TT::XROWS * 128) >> 4) + 2 * (j & 3)),
                              idesc, 0u);
                tc_commit(&bars->a_empty[as]);
                tc_commit(&bars->tmem_full[ts]);
                TCQ_TRACE(5, g);
                ready = n0 && n1 && n2;
            }
        }
    } else if (warp >= 4 && warp < 4 + TCQ_UNPACK_WARPS) {
        // ---------------- unpacking: two groups of four warps take alternate stages; thread = row, both sub-tiles ----------------
        const int ut = tid - 128;
        const int grp = ut >> 7;
        const int r = ut & (TCQ_ROWS - 1);
        TcqRing rr, ar, sr;
        int kc = kc0;
        if (grp == 1) {  // first stage of this group is g = 1
            rr.next(NR);
            ar.next(NA);
            sr.next(TCQ_SC_STAGES);
            if (++kc == kc1) kc = kc0;
        }
        bool ok = true;
        for (int g = grp; g < nstages; g += 2) {
            ok = mbar_wait3_bounded(&bars->raw_full[rr.i], rr.ph, &bars->a_empty[ar.i], ar.ph ^ 1, &bars->sc_empty[sr.i], sr.ph ^ 1);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, 1000 + g);
                break;
            }
            if ((ut & 127) == 0) TCQ_TRACE(2, g);
            if (r < TH) {
                const uint32_t rb = smem_u32(raw_stages + (size_t)rr.i * raw_bytes) + (uint32_t)r * TT::PITCH;
                const uint32_t a_sub = smem_u32(a_stages + (size_t)ar.i * a_bytes);
                const uint32_t sc = smem_u32(sc_stages + (size_t)sr.i * TCQ_SC_BYTES) + (uint32_t)r * TCQ_SC_PITCH;
                TcqUnpack<TYPE>::run(rb, kc, 0, r, a_sub, sc);
                TcqUnpack<TYPE>::run(rb, kc, 1, r, a_sub + sub_bytes, sc);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars->a_full[ar.i]);
                mbar_arrive(&bars->sc_full[sr.i]);
                mbar_arrive(&bars->raw_empty[rr.i]);
            }
            if ((ut & 127) == 0) TCQ_TRACE(3, g);
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                rr.next(NR);
                ar.next(NA);
                sr.next(TCQ_SC_STAGES);
                if (++kc == kc1) kc = kc0;
            }
        }
    } else if (warp >= 4 + TCQ_UNPACK_WARPS) {
        // ---------------- scaling: thread = weight row (TMEM lane); the row's eight blocks of a stage are split over the
        // four warps that may read its lanes (two blocks each, all activation rows) ----------------
        const int sw = warp - (4 + TCQ_UNPACK_WARPS);
        const int quarter = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp % 4)
        const int tg = sw >> 2;        // blocks 2 tg, 2 tg + 1
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float acc[TOK];
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc[t] = 0.0f;
        TcqRing xr, sr, tr;
        int kc = kc0, t = 0;
        bool ok = true;
        for (int g = 0; g < nstages; ++g) {
            ok = mbar_wait3_bounded(&bars->tmem_full[tr.i], tr.ph, &bars->sc_full[sr.i], sr.ph, &bars->x_full[xr.i], xr.ph);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) {
                if (lane == 0) record_failure(p.status, STATUS_WAIT_MMA_TIMEOUT, g);
                break;
            }
            tc_fence_after();
            if (sw == 0 && lane == 0) TCQ_TRACE(6, g);
            {
                const uint32_t col0 = lane_base + tr.i * L::BUF_COLS + 2 * tg * L::NCOL;
                constexpr bool TWO_PASSES = TYPE == TYPE_Q6_K && TOK == 16;  // four 16-register loads at once would spill
                uint32_t I0[TOK], I1[TOK], O0[TOK], O1[TOK];
                tcq_tmem_ld<TOK>(col0, I0);
                if constexpr (TYPE == TYPE_Q6_K) tcq_tmem_ld<TOK>(col0 + TCQ_TOKENS, O0);
                if constexpr (!TWO_PASSES) {
                    tcq_tmem_ld<TOK>(col0 + L::NCOL, I1);
                    if constexpr (TYPE == TYPE_Q6_K) tcq_tmem_ld<TOK>(col0 + L::NCOL + TCQ_TOKENS, O1);
                }
                const uint32_t sca = smem_u32(sc_stages + (size_t)sr.i * TCQ_SC_BYTES) + (uint32_t)r * TCQ_SC_PITCH;
                const uint32_t dsb = smem_u32(x_stages + (size_t)xr.i * L::X_BYTES + TT::XROWS * TCQ_KC) + (uint32_t)(2 * tg) * (TCQ_TOKENS * 8);
                float s00, s01, s10, s11;  // block 2 tg: s00, s01; block 2 tg + 1: s10, s11
                if constexpr (TYPE == TYPE_Q4_K) {
                    const uint2 a = lds64(sca + 8 * tg), b = lds64(sca + 32 + 8 * tg);
                    s00 = __uint_as_float(a.x); s10 = __uint_as_float(a.y);
                    s01 = __uint_as_float(b.x); s11 = __uint_as_float(b.y);
                } else if constexpr (TYPE == TYPE_Q8_0) {
                    const uint2 a = lds64(sca + 8 * tg);
                    s00 = __uint_as_float(a.x); s10 = __uint_as_float(a.y);
                    s01 = s11 = 0.0f;
                } else {
                    const uint4 a = lds128(sca + 16 * tg);
                    s00 = __uint_as_float(a.x); s01 = __uint_as_float(a.y); s10 = __uint_as_float(a.z); s11 = __uint_as_float(a.w);
                }
                tmem_ld_wait();
                tcq_scale_block<TYPE, TOK>(I0, O0, s00, s01, dsb, acc);
                if constexpr (TWO_PASSES) {
                    tcq_tmem_ld<TOK>(col0 + L::NCOL, I0);
                    tcq_tmem_ld<TOK>(col0 + L::NCOL + TCQ_TOKENS, O0);
                    tmem_ld_wait();
                    tcq_scale_block<TYPE, TOK>(I0, O0, s10, s11, dsb + TCQ_TOKENS * 8, acc);
                } else {
                    tcq_scale_block<TYPE, TOK>(I1, O1, s10, s11, dsb + TCQ_TOKENS * 8, acc);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&bars->tmem_empty[tr.i]);
                mbar_arrive(&bars->sc_empty[sr.i]);
                mbar_arrive(&bars->x_empty[xr.i]);
            }
            if (sw == 0 && lane == 0) TCQ_TRACE(7, g);
            xr.next(XS);
            sr.next(TCQ_SC_STAGES);
            tr.next(TB);
            if (++kc == kc1) {
                kc = kc0;
                // ---------------- end of a tile: the four warps of a row add up through shared memory in a fixed
                // order (block pairs 0, 1, 2, 3: results do not depend on timing), the last one stores ----------------
                float* o = out_buf + r * TCQ_TOKENS;
                if (tg == 0) {
                    // the previous tile's sums must have been read before they are overwritten
                    ok = t == 0 || mbar_wait_bounded(&bars->comb[3], (t - 1) & 1);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) {
                        if (lane == 0) record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, 3000 + t);
                        break;
                    }
#pragma unroll
                    for (int tt = 0; tt < TOK; ++tt) o[tt] = acc[tt];
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->comb[0]);
                } else {
                    ok = __all_sync(0xffffffffu, mbar_wait_bounded(&bars->comb[tg - 1], t & 1));
                    if (!ok) {
                        if (lane == 0) record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, 4000 + t);
                        break;
                    }
#pragma unroll
                    for (int tt = 0; tt < TOK; ++tt) acc[tt] = o[tt] + acc[tt];
                    if (tg < 3) {
#pragma unroll
                        for (int tt = 0; tt < TOK; ++tt) o[tt] = acc[tt];
                    } else {
                        const int grow = row0 + t * TH + r;
                        const bool row_ok = r < TH && grow < row1;
                        dst_t* y = reinterpret_cast<dst_t*>(p.y) + grow;
                        if (p.ksplit <= 1) {
                            if (row_ok) {
#pragma unroll
                                for (int tt = 0; tt < TOK; ++tt)
                                    if (tt < p.M) y[(size_t)tt * p.ldy] = from_float<dst_t>(acc[tt]);
                            }
                        } else {
                            // this split's share of the row's outputs -> global; the last split to arrive for these 32
                            // rows adds all shares in split order (timing does not change the result) and stores
                            const int split = cta % p.ksplit;
                            float* mine = p.partial + ((size_t)split * TCQ_TOKENS) * p.N + grow;
                            if (row_ok) {
#pragma unroll
                                for (int tt = 0; tt < TOK; ++tt)
                                    if (tt < p.M) mine[(size_t)tt * p.N] = acc[tt];
                            }
                            __threadfence();
                            __syncwarp();
                            unsigned int arrived = 0;
                            if (lane == 0) arrived = atomicAdd(p.counters + (cta / p.ksplit) * 4 + quarter, 1u);
                            arrived = __shfl_sync(0xffffffffu, arrived, 0);
                            if (arrived == (unsigned int)p.ksplit - 1u) {
                                __threadfence();
                                if (row_ok) {
#pragma unroll
                                    for (int tt = 0; tt < TOK; ++tt) {
                                        if (tt < p.M) {
                                            float v = 0.0f;
                                            for (int sp = 0; sp < p.ksplit; ++sp)
                                                v += __ldcg(p.partial + ((size_t)sp * TCQ_TOKENS + tt) * p.N + grow);
                                            y[(size_t)tt * p.ldy] = from_float<dst_t>(v);
                                        }
                                    }
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->comb[tg]);
                }
#pragma unroll
                for (int tt = 0; tt < TOK; ++tt) acc[tt] = 0.0f;
                ++t;
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
// workspace: int8 activations [xrows][K] | float2 scales [K / 32][16] | K-split counters | K-split partial outputs
static size_t tcq_quant_bytes(int type, int K) {
    const size_t xrows = type == TYPE_Q6_K ? 32 : 16;
    return xrows * (size_t)K + (size_t)(K / 32) * TCQ_TOKENS * sizeof(float2);
}
size_t gemv_tc_workspace_bytes(int type, int K) {
    return ((tcq_quant_bytes(type, K) + 255) & ~(size_t)255) + TCQ_COUNTERS * sizeof(unsigned int) + TCQ_PARTIAL_BYTES;
}

template <int TYPE, typename T, int TOK, bool REF_ACTS = false>
static int launch_gemv_tc_i8_tok(const CUtensorMap& map_w, const CUtensorMap& map_x, const TcqParams& p, int grid, int smem_bytes,
                                 cudaStream_t s, bool after_quantizer = false) {
    auto kernel = gemv_tc_i8_kernel<TYPE, T, TOK, REF_ACTS>;
    static PerDeviceOnce configured;  // per instantiation and device
    const cudaError_t attr_err =
        configured.run([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TCQ_SMEM_LIMIT); });
    if (attr_err != cudaSuccess) return (int)attr_err;
    // `after_quantizer`: the launch directly before this one on the stream is this file's quantizer, which lets its
    // dependents start early; the two overlap safely because the quantizer writes nothing this kernel reads before its wait
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(TCQ_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_bytes;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = after_quantizer ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, map_w, map_x, p);
}

// Row split, K split and ring depths for a shape; fills p.{ksplit, tile_rows, rows_per_cta, rows_extra, a_stages,
// raw_stages}. Returns 0 or B200Q_ERR_UNSUPPORTED.
template <int TYPE>
static int tcq_plan(TcqParams& p, int N, int K, bool allow_ksplit, int& grid, int& smem_bytes) {
    using TT = TcqType<TYPE>;
    using L = TcqLayout<TYPE>;
    const int sms = runtime_info().sm_count < TCQ_MAX_CTAS ? runtime_info().sm_count : TCQ_MAX_CTAS;
    const int nkc = K / TCQ_KC;
    const int row_tiles = (N + TCQ_ROWS - 1) / TCQ_ROWS;
    p.ksplit = 1;
    if (allow_ksplit && 2 * row_tiles <= sms && nkc >= 4 && runtime_info().tc_ksplit) {
        // few rows: full-height tiles, K shared out so that most SMs get a unit of at least two stages
        int ks = sms / row_tiles;
        if (ks > nkc / 2) ks = nkc / 2;
        p.ksplit = ks;
    }
    if (p.ksplit > 1) {
        p.tile_rows = N < TCQ_ROWS ? ((N + 7) & ~7) : TCQ_ROWS;
        p.rows_per_cta = p.tile_rows;
        p.rows_extra = 0;
        grid = row_tiles * p.ksplit;
    } else {
        grid = sms;
        if (grid > N) grid = N;
        p.rows_per_cta = N / grid;
        p.rows_extra = N % grid;
        const int max_rows = p.rows_per_cta + (p.rows_extra ? 1 : 0);
        const int tiles = (max_rows + TCQ_ROWS - 1) / TCQ_ROWS;
        p.tile_rows = (((max_rows + tiles - 1) / tiles) + 7) & ~7;
    }
    // ring depths: prefer four A stages if at least three packed-row stages still fit, else three (two at worst)
    const int a_bytes = 2 * p.tile_rows * 128, raw_bytes = (p.tile_rows * TT::PITCH + 127) & ~127;
    const int room = TCQ_SMEM_LIMIT - L::FIXED;
    p.a_stages = 4;
    while (p.a_stages > 2 && (room - p.a_stages * a_bytes) / raw_bytes < (p.a_stages == 4 ? 3 : 2)) --p.a_stages;
    p.raw_stages = (room - p.a_stages * a_bytes) / raw_bytes;
    if (p.raw_stages > 8) p.raw_stages = 8;
    if (p.raw_stages < 2) return B200Q_ERR_UNSUPPORTED;
    smem_bytes = L::FIXED + p.a_stages * a_bytes + p.raw_stages * raw_bytes;
    return 0;
}

// 2-D tensor map over the packed weight bytes: boxes of tile_rows x one 256-k chunk
template <int TYPE>
static int tcq_encode_w(CUtensorMap& map_w, const void* w, int N, int K, int tile_rows) {
    using TT = TcqType<TYPE>;
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return B200Q_ERR_UNSUPPORTED;
    const int row_bytes = K / type_block_elems(TYPE) * type_block_bytes(TYPE);
    const bool u16 = TYPE == TYPE_Q8_0;  // a 272-byte chunk is more than 256 one-byte elements
    const cuuint64_t dims[2] = {(cuuint64_t)(u16 ? row_bytes / 2 : row_bytes), (cuuint64_t)N};
    const cuuint32_t box[2] = {(cuuint32_t)(u16 ? TT::PITCH / 2 : TT::PITCH), (cuuint32_t)tile_rows};
    CUresult r = encode_tiled_2d_cached(&map_w, u16 ? CU_TENSOR_MAP_DATA_TYPE_UINT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, w, dims,
                                        (cuuint64_t)row_bytes, box, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    return r == CUDA_SUCCESS ? 0 : B200Q_ERR_INVALID;
}

template <int TYPE, typename T>
static int launch_gemv_tc_i8(const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, void* workspace, cudaStream_t s) {
    using TT = TcqType<TYPE>;
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return B200Q_ERR_UNSUPPORTED;
    int8_t* q = static_cast<int8_t*>(workspace);
    float2* ds = reinterpret_cast<float2*>(q + (size_t)TT::XROWS * K);

    TcqParams p{};
    p.y = y;
    p.ds = reinterpret_cast<const uint8_t*>(ds);
    p.M = M;
    p.N = N;
    p.K = K;
    p.ldy = ldy;
    p.status = status_ptr();
    {
        int slots = 0;
        p.trace = trace_buffer(&slots);
        p.trace_stages = slots / 8;
    }
    uint8_t* after = static_cast<uint8_t*>(workspace) + ((tcq_quant_bytes(TYPE, K) + 255) & ~(size_t)255);
    p.counters = reinterpret_cast<unsigned int*>(after);
    p.partial = reinterpret_cast<float*>(after + TCQ_COUNTERS * sizeof(unsigned int));
    int grid = 0, smem_bytes = 0;
    int rc = tcq_plan<TYPE>(p, N, K, true, grid, smem_bytes);
    if (rc != 0) return rc;
    CUtensorMap map_w, map_x;
    rc = tcq_encode_w<TYPE>(map_w, w, N, K, p.tile_rows);
    if (rc != 0) return rc;
    {
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)TT::XROWS};
        const cuuint32_t box[2] = {128, (cuuint32_t)TT::XROWS};
        CUresult r = encode_tiled_2d_cached(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, q, dims, (cuuint64_t)K, box, CU_TENSOR_MAP_SWIZZLE_128B,
                                            CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
        if (r != CUDA_SUCCESS) return B200Q_ERR_INVALID;
    }

    tcq_quantize_kernel<T, TYPE == TYPE_Q6_K><<<K / 32, dim3(32, TCQ_TOKENS), 0, s>>>(static_cast<const T*>(x), q, ds, K, M, ldx, p.counters);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;

    if (M <= 4) return launch_gemv_tc_i8_tok<TYPE, T, 4>(map_w, map_x, p, grid, smem_bytes, s, true);
    if (M <= 8) return launch_gemv_tc_i8_tok<TYPE, T, 8>(map_w, map_x, p, grid, smem_bytes, s, true);
    return launch_gemv_tc_i8_tok<TYPE, T, 16>(map_w, map_x, p, grid, smem_bytes, s, true);
}

// ---------------------------------------------------------------------------------------------
// The reference tier's own pair of launchers (crates/inference-quant/src/gguf/ffi.rs:631-652,954-998): the host
// quantizes with launch_mmvq_tc_quantize_<elem> into ITS scratch (288 bytes per 32-value block and 8-row half,
// fast_mmvq.rs:94,1898-1902) and hands that to launch_mmvq_tc_gguf_<type>_<elem>_plain. The matvec is the kernel
// above with REF_ACTS: one warp re-lays the fragments out stage by stage, so nothing beyond the host's scratch is
// needed; without a workspace for partial outputs the split along K is off. Shapes the TMA path cannot take (packed
// rows that are not a multiple of 16 bytes, unaligned weights) go to a plain one-warp-per-row kernel on the same layout.
// ---------------------------------------------------------------------------------------------
template <int TYPE, typename dst_t>
__global__ void __launch_bounds__(256) gemv_tc_ref_simple_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ acts,
                                                                 dst_t* __restrict__ dst, int K, int N, int stride_dst, int M) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= N) return;
    const int nb = K / 32;
    const uint8_t* rp = w + (size_t)row * (K / 256) * type_block_bytes(TYPE);
    float acc[TCQ_TOKENS];
#pragma unroll
    for (int t = 0; t < TCQ_TOKENS; ++t) acc[t] = 0.0f;
    for (int kb = lane; kb < nb; kb += 32) {
        int wq[32];
        float s0 = 0.0f, s1 = 0.0f, mn = 0.0f;  // Q4_K: s0 = d * sc, mn = dmin * m; Q6_K: s0, s1 = d * sc of the two halves
        const int sblk = kb >> 3;
        if (TYPE == TYPE_Q4_K) {
            const int j = kb & 7;
            const uint8_t* sb = rp + (size_t)sblk * Q4_K_BYTES;
            const uint8_t* q = sb + 4;
            int sc, m;
            if (j < 4) { sc = q[j] & 63; m = q[j + 4] & 63; }
            else { sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4); m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4); }
            s0 = half_bits_to_float((uint32_t)sb[0] | ((uint32_t)sb[1] << 8)) * (float)sc;
            mn = half_bits_to_float((uint32_t)sb[2] | ((uint32_t)sb[3] << 8)) * (float)m;
            const uint8_t* qs = sb + 16 + 32 * (j >> 1);
            for (int l = 0; l < 32; ++l) wq[l] = (j & 1) ? (qs[l] >> 4) : (qs[l] & 0xF);
        } else {
            const int n = (kb >> 2) & 1, qd = kb & 3;
            const uint8_t* sb = rp + (size_t)sblk * Q6_K_BYTES;
            const uint8_t* ql = sb + 64 * n + 32 * (qd & 1);
            const uint8_t* qh = sb + 128 + 32 * n;
            for (int l = 0; l < 32; ++l) {
                const int lo = (qd & 2) ? (ql[l] >> 4) : (ql[l] & 0xF);
                wq[l] = (lo | (((qh[l] >> (2 * qd)) & 3) << 4)) - 32;
            }
            const float d = half_bits_to_float((uint32_t)sb[208] | ((uint32_t)sb[209] << 8));
            s0 = d * (float)(int)(int8_t)sb[192 + 8 * n + 2 * qd];
            s1 = d * (float)(int)(int8_t)sb[192 + 8 * n + 2 * qd + 1];
        }
        for (int t = 0; t < M; ++t) {
            const uint8_t* base = acts + (size_t)(t >> 3) * nb * TCQ_REF_BLOCK_BYTES;
            const int r = t & 7;
            const int8_t* frag = reinterpret_cast<const int8_t*>(base) + (size_t)kb * 256 + (4 * r) * 8;
            const float xd = __half2float(reinterpret_cast<const __half*>(base + (size_t)nb * 256)[kb * 8 + r]);
            int d0 = 0, d1 = 0;
            for (int l = 0; l < 16; ++l) d0 += wq[l] * (int)frag[(l >> 2) * 8 + (l & 3)];
            for (int l = 16; l < 32; ++l) d1 += wq[l] * (int)frag[((l - 16) >> 2) * 8 + 4 + (l & 3)];
            if (TYPE == TYPE_Q4_K) {
                const int sum = (int)reinterpret_cast<const int16_t*>(base + (size_t)nb * 256 + (size_t)nb * 16)[kb * 8 + r];
                acc[t] += s0 * (xd * (float)(d0 + d1)) - mn * (xd * (float)sum);
            } else {
                acc[t] += xd * (s0 * (float)d0 + s1 * (float)d1);
            }
        }
    }
    for (int t = 0; t < M; ++t) {
        const float v = warp_sum(acc[t]);
        if (lane == 0) dst[(size_t)t * stride_dst + row] = from_float<dst_t>(v);
    }
}

template <typename T>
static int launch_tcq_ref_quantize(const void* x, void* vy, int kx, int num_rows, cudaStream_t s) {
    if (kx <= 0 || num_rows <= 0) return 0;
    const dim3 grid((unsigned)((kx + 31) / 32), (unsigned)((num_rows + 7) / 8), 1);
    tcq_ref_quantize_kernel<T><<<grid, dim3(32, 8, 1), 0, s>>>(static_cast<const T*>(x), static_cast<uint8_t*>(vy), kx, num_rows);
    return (int)cudaGetLastError();
}

template <int TYPE, typename T>
static int launch_gemv_tc_ref(const void* w, const void* vy, void* dst, int K, int N, int stride_col_dst, int b, cudaStream_t s) {
    if (N <= 0 || K <= 0 || b <= 0) return 0;
    if (b > TCQ_TOKENS || K % TCQ_KC != 0) return B200Q_ERR_UNSUPPORTED;
    const int row_bytes = K / 256 * type_block_bytes(TYPE);
    const bool tma_ok = reinterpret_cast<uintptr_t>(w) % 16 == 0 && row_bytes % 16 == 0 && encode_tiled_fn() != nullptr;
    if (!tma_ok) {
        gemv_tc_ref_simple_kernel<TYPE, T><<<(N + 7) / 8, 256, 0, s>>>(static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(vy),
                                                                      static_cast<T*>(dst), K, N, stride_col_dst, b);
        return (int)cudaGetLastError();
    }
    TcqParams p{};
    p.y = dst;
    p.M = b;
    p.N = N;
    p.K = K;
    p.ldy = stride_col_dst;
    p.status = status_ptr();
    p.ref_acts = static_cast<const uint8_t*>(vy);
    p.ref_halves = (b + 7) / 8;
    int grid = 0, smem_bytes = 0;
    int rc = tcq_plan<TYPE>(p, N, K, false, grid, smem_bytes);
    if (rc != 0) return rc;
    CUtensorMap map_w;
    rc = tcq_encode_w<TYPE>(map_w, w, N, K, p.tile_rows);
    if (rc != 0) return rc;
    // (the activation map parameter is not read by the REF_ACTS kernels)
    if (b <= 4) return launch_gemv_tc_i8_tok<TYPE, T, 4, true>(map_w, map_w, p, grid, smem_bytes, s);
    if (b <= 8) return launch_gemv_tc_i8_tok<TYPE, T, 8, true>(map_w, map_w, p, grid, smem_bytes, s);
    return launch_gemv_tc_i8_tok<TYPE, T, 16, true>(map_w, map_w, p, grid, smem_bytes, s);
}

int gemv_tc_dispatch(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, void* workspace,
                     cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (M > TCQ_TOKENS || K <= 0 || K % TCQ_KC != 0) return B200Q_ERR_UNSUPPORTED;
    const int row_bytes = K / type_block_elems(type) * type_block_bytes(type);
    if (reinterpret_cast<uintptr_t>(w) % 16 != 0 || row_bytes % 16 != 0) return B200Q_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(workspace) % 128 != 0) return B200Q_ERR_INVALID;
#define B200Q_TCQ_CASE(TYPE)                                                                                              \
    if (type == TYPE) {                                                                                                   \
        if (elem == ELEM_BF16) return launch_gemv_tc_i8<TYPE, __nv_bfloat16>(w, x, y, M, N, K, ldx, ldy, workspace, s);   \
        if (elem == ELEM_F16) return launch_gemv_tc_i8<TYPE, __half>(w, x, y, M, N, K, ldx, ldy, workspace, s);           \
        if (elem == ELEM_F32) return launch_gemv_tc_i8<TYPE, float>(w, x, y, M, N, K, ldx, ldy, workspace, s);            \
        return B200Q_ERR_UNSUPPORTED;                                                                                     \
    }
    B200Q_TCQ_CASE(TYPE_Q4_K)
    B200Q_TCQ_CASE(TYPE_Q6_K)
    B200Q_TCQ_CASE(TYPE_Q8_0)
#undef B200Q_TCQ_CASE
    return B200Q_ERR_UNSUPPORTED;
}

}  // namespace b200q

// The reference's symbols; void, asynchronous, allocation-free. `cfg` selects among the reference kernel's own launch
// shapes (mmvq_tc_k.cuh:352-375) and has no meaning for this kernel.
#define B200Q_TC_QUANTIZE(tag, T)                                                                                          \
    extern "C" void launch_mmvq_tc_quantize_##tag(const void* x, void* vy, int kx, int num_rows, void* stream) {          \
        b200q::note_launch_status(b200q::launch_tcq_ref_quantize<T>(x, vy, kx, num_rows, (cudaStream_t)stream));           \
    }
B200Q_TC_QUANTIZE(bf16, __nv_bfloat16)
B200Q_TC_QUANTIZE(f16, __half)
B200Q_TC_QUANTIZE(f32, float)
#undef B200Q_TC_QUANTIZE

#define B200Q_TC_PLAIN(type_tag, TYPE, tag, T)                                                                             \
    extern "C" void launch_mmvq_tc_gguf_##type_tag##_##tag##_plain(const void* vx, const void* vy, void* dst, int ncols_x,  \
                                                                   int nrows_x, int stride_col_dst, int b_size, int cfg,   \
                                                                   void* stream) {                                         \
        (void)cfg;                                                                                                         \
        b200q::note_launch_status(                                                                                         \
            b200q::launch_gemv_tc_ref<TYPE, T>(vx, vy, dst, ncols_x, nrows_x, stride_col_dst, b_size, (cudaStream_t)stream)); \
    }
B200Q_TC_PLAIN(q4_k, b200q::TYPE_Q4_K, bf16, __nv_bfloat16)
B200Q_TC_PLAIN(q4_k, b200q::TYPE_Q4_K, f16, __half)
B200Q_TC_PLAIN(q4_k, b200q::TYPE_Q4_K, f32, float)
B200Q_TC_PLAIN(q6_k, b200q::TYPE_Q6_K, bf16, __nv_bfloat16)
B200Q_TC_PLAIN(q6_k, b200q::TYPE_Q6_K, f16, __half)
B200Q_TC_PLAIN(q6_k, b200q::TYPE_Q6_K, f32, float)
#undef B200Q_TC_PLAIN

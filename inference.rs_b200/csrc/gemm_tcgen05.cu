// Prefill GEMM: Y[m][n] = sum_k X[m][k] * W[n][k] for packed Q8_0 / Q4_K / Q6_K weights (GGUF layout) and M >= 17
// bf16 / f16 activation rows, f32 accumulation, output in the activation type. Takes the place of the reference's
// tiled int8 path `mul_mat_q` (crates/inference-quant/kernels/cuda/mmq_gguf/mmq_gguf.cuh:3632-3875, host side
// crates/inference-quant/src/gguf/fast_mmq.rs:604-715) with a tile GEMM on the 5th-generation tensor cores:
//
//   * A operand = activations, 128 tokens x 64 k per stage, brought in by TMA (cp.async.bulk.tensor, 128-byte swizzle);
//   * B operand = weights, dequantized by eight warps from the packed blocks straight into the same K-major
//     128-byte-swizzled shared-memory layout as bf16 / f16 (scale and min folded in f32, one rounding), made visible
//     to the tensor core with a proxy fence; activations are NOT quantized, so the only error is the weights' own;
//   * tcgen05.mma (kind::f16, M = 128, N = 128, K = 16) issued by one thread, accumulators in TMEM (one 128-column
//     block per 128-token sub-tile, 1 or 2 sub-tiles per CTA), completion signalled with tcgen05.commit on mbarriers;
//   * epilogue: tcgen05.ld 32 lanes x 32 columns per warp, convert, 64-byte stores per token row.
//
// Every wait is bounded; a wait that gives up records a code in the device status word, work is skipped, and the
// kernel still frees its TMEM columns before it returns.
#include <cuda.h>

#include "common.cuh"
#include "runtime.h"
#include "tcgen05.cuh"

namespace b200q {

constexpr int GEMM_BM = 128;       // tokens per sub-tile = TMEM lanes
constexpr int GEMM_BN = 128;       // weight rows per tile = TMEM columns per sub-tile
constexpr int GEMM_BK = 64;        // k per stage: one 128-byte swizzled row of 16-bit elements
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_DEQ_WARPS = 8;  // warps 4..11
constexpr int GEMM_THREADS = 32 * (4 + GEMM_DEQ_WARPS);
constexpr int GEMM_A_BYTES = GEMM_BM * GEMM_BK * 2;  // 16 KB per sub-tile and stage
constexpr int GEMM_B_BYTES = GEMM_BN * GEMM_BK * 2;  // 16 KB per stage

struct GemmParams {
    const uint8_t* w;  // packed weights [N][K / block]
    void* y;           // [M][ldy]
    int M, N, K;
    int ldy;
    int row_bytes;
    unsigned int* status;
    // AQ kernels: activations arrive already quantized, as the reference's prefill quantizer lays them out (144-byte
    // blocks of 128 values of one token: 16 bytes of scales, then 128 int8; block (k / 128) * M + token;
    // crates/inference-quant/kernels/cuda/mmq_gguf/mmq_gguf.cuh:70-89, mmq_quantize.cu:126-131)
    const uint8_t* aq;
    int aq_ds4;  // scales are four half2 (d, sum) instead of four f32 d
};

template <typename T> struct ElemFormat;  // tcgen05 kind::f16 operand format code
template <> struct ElemFormat<__half> { static constexpr int value = 0; };
template <> struct ElemFormat<__nv_bfloat16> { static constexpr int value = 1; };

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------------------------------------
// Dequantization of one unit = 32 consecutive k of one weight row (half h of a 64-wide k block) into 64 bytes of the
// B stage. The packed blocks are read straight from global memory (L2 serves the re-reads of other token tiles).
// ---------------------------------------------------------------------------------------------
template <int N>
__device__ __forceinline__ void ldg_words_u16aligned(const uint8_t* p, uint32_t (&out)[N]) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    const uint32_t shift = (uint32_t)(a & 2u) * 8u;
    const uint32_t* base = reinterpret_cast<const uint32_t*>(a & ~(uintptr_t)3);
    uint32_t w[N + 1];
#pragma unroll
    for (int i = 0; i <= N; ++i) w[i] = __ldg(base + i);
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = __funnelshift_r(w[i], w[i + 1], shift);
}
__device__ __forceinline__ uint32_t ldg_u16(const uint8_t* p) { return (uint32_t)__ldg(reinterpret_cast<const unsigned short*>(p)); }

// byte b (0..255) -> float, exactly, without the conversion unit
__device__ __forceinline__ float byte_to_float(uint32_t b) { return __uint_as_float(0x4B000000u | b) - 8388608.0f; }
// byte `idx` of w as the float 2^23 + byte (one byte-permute); subtract 2^23 (+ an offset) to get the value
template <int idx> __device__ __forceinline__ float byte_as_magic(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650 | idx));
}

template <typename T>
__device__ __forceinline__ void store_unit(uint32_t stage_addr, int r, int h, const float (&v)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        sts128(b_chunk_addr(stage_addr, r, 4 * h + i), pack2<T>(v[8 * i], v[8 * i + 1]), pack2<T>(v[8 * i + 2], v[8 * i + 3]),
               pack2<T>(v[8 * i + 4], v[8 * i + 5]), pack2<T>(v[8 * i + 6], v[8 * i + 7]));
    }
}

template <int TYPE> struct Dequant;

// Q4_K: k block kb = chunk c = kb & 3 of superblock kb >> 2; half h is sub-block 2c + h (low / high nibbles of the
// same 32 bytes). value = d * sc * q - dmin * m (crates/inference-tensor/src/quantized/k_quants.rs:2096-2123).
template <> struct Dequant<TYPE_Q4_K> {
    uint4 hdr, q0, q1;
    __device__ __forceinline__ void load(const uint8_t* row, int kb, int) {
        const uint8_t* sb = row + (size_t)(kb >> 2) * Q4_K_BYTES;
        hdr = __ldg(reinterpret_cast<const uint4*>(sb));
        q0 = __ldg(reinterpret_cast<const uint4*>(sb + 16 + 32 * (kb & 3)));
        q1 = __ldg(reinterpret_cast<const uint4*>(sb + 32 + 32 * (kb & 3)));
    }
    __device__ __forceinline__ void values(int kb, int h, float (&v)[32]) const {
        const int j = 2 * (kb & 3) + h;
        uint32_t sc, m;
        if (j < 4) {
            sc = ((hdr.y >> (8 * j)) & 0x3fu);
            m = ((hdr.z >> (8 * j)) & 0x3fu);
        } else {
            const int jj = j - 4;
            const uint32_t lo = (hdr.w >> (8 * jj)) & 0xffu;
            sc = (lo & 0xfu) | ((((hdr.y >> (8 * jj)) & 0xffu) >> 6) << 4);
            m = (lo >> 4) | ((((hdr.z >> (8 * jj)) & 0xffu) >> 6) << 4);
        }
        const float dl = half_bits_to_float(hdr.x) * byte_to_float(sc);
        const float ml = half_bits_to_float(hdr.x >> 16) * byte_to_float(m);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const int sh = 4 * h;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t nib = (w[i] >> sh) & 0x0f0f0f0fu;  // four quants, one per byte
            v[4 * i + 0] = fmaf(dl, byte_as_magic<0>(nib) - 8388608.0f, -ml);
            v[4 * i + 1] = fmaf(dl, byte_as_magic<1>(nib) - 8388608.0f, -ml);
            v[4 * i + 2] = fmaf(dl, byte_as_magic<2>(nib) - 8388608.0f, -ml);
            v[4 * i + 3] = fmaf(dl, byte_as_magic<3>(nib) - 8388608.0f, -ml);
        }
    }
};

// Q6_K: k block kb: superblock kb >> 2, half n = (kb & 3) >> 1, pair p = kb & 1; unit h is quarter qd = 2p + h:
// ql[64n + 32h + l] nibble p, qh[32n + l] bits 2qd, scale[8n + 2qd + l/16]; value = d * sc * (q - 32)
// (crates/inference-tensor/src/quantized/k_quants.rs:2649-2680).
template <> struct Dequant<TYPE_Q6_K> {
    uint32_t ql[8], qh[8];
    uint32_t sc2, dbits;
    __device__ __forceinline__ void load(const uint8_t* row, int kb, int h) {
        const uint8_t* sb = row + (size_t)(kb >> 2) * Q6_K_BYTES;
        const int n = (kb & 3) >> 1, qd = 2 * (kb & 1) + h;
        ldg_words_u16aligned<8>(sb + 64 * n + 32 * h, ql);
        ldg_words_u16aligned<8>(sb + 128 + 32 * n, qh);
        sc2 = ldg_u16(sb + 192 + 8 * n + 2 * qd);
        dbits = ldg_u16(sb + 208);
    }
    __device__ __forceinline__ void values(int kb, int h, float (&v)[32]) const {
        const int p = kb & 1, qd = 2 * p + h;
        const float d = half_bits_to_float(dbits);
        const float s0 = d * (float)(int)(int8_t)(sc2 & 0xffu), s1 = d * (float)(int)(int8_t)(sc2 >> 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // four 6-bit quants, one per byte: low nibble | two high bits << 4
            const uint32_t q4 = ((ql[i] >> (4 * p)) & 0x0f0f0f0fu) | (((qh[i] >> (2 * qd)) & 0x03030303u) << 4);
            const float sc = i < 4 ? s0 : s1;
            v[4 * i + 0] = sc * (byte_as_magic<0>(q4) - 8388640.0f);  // 2^23 + 32
            v[4 * i + 1] = sc * (byte_as_magic<1>(q4) - 8388640.0f);
            v[4 * i + 2] = sc * (byte_as_magic<2>(q4) - 8388640.0f);
            v[4 * i + 3] = sc * (byte_as_magic<3>(q4) - 8388640.0f);
        }
    }
};

// Q8_0: unit h of k block kb is block 2 kb + h: f16 d, 32 int8; value = d * q.
template <> struct Dequant<TYPE_Q8_0> {
    uint32_t w[9];
    __device__ __forceinline__ void load(const uint8_t* row, int kb, int h) {
        ldg_words_u16aligned<9>(row + (size_t)(2 * kb + h) * Q8_0_BYTES, w);  // bytes 0..35 (34 used)
    }
    __device__ __forceinline__ void values(int, int, float (&v)[32]) const {
        const float d = half_bits_to_float(w[0]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            // bytes 2 + 4i .. 5 + 4i, flipped to unsigned (q + 128)
            const uint32_t q = __funnelshift_r(w[i], w[i + 1], 16) ^ 0x80808080u;
            v[4 * i + 0] = d * (byte_as_magic<0>(q) - 8388736.0f);  // 2^23 + 128
            v[4 * i + 1] = d * (byte_as_magic<1>(q) - 8388736.0f);
            v[4 * i + 2] = d * (byte_as_magic<2>(q) - 8388736.0f);
            v[4 * i + 3] = d * (byte_as_magic<3>(q) - 8388736.0f);
        }
    }
};

// ---------------------------------------------------------------------------------------------
// The kernel: one CTA computes a (MT * 128 tokens) x (128 weight rows) tile over the whole K.
//   warp 0    TMA producer of the activation sub-tiles
//   warp 1    tcgen05.mma issuer
//   warp 2    TMEM allocation / release
//   warps 4+  weight dequantization into the B stages, then the epilogue
// ---------------------------------------------------------------------------------------------
struct GemmBarriers {
    uint64_t full_a[GEMM_STAGES];
    uint64_t full_b[GEMM_STAGES];
    uint64_t empty[GEMM_STAGES];
    uint64_t tmem_full;
    uint32_t tmem_base;
    uint32_t failed;
};

template <int TYPE, typename T, int MT>
__global__ void __launch_bounds__(GEMM_THREADS, 1) gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    extern __shared__ uint8_t gemm_smem_raw[];
    // operand stages need 1024-byte alignment for the 128-byte swizzle
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* a_stages = smem;                                        // [S][MT][16 KB]
    uint8_t* b_stages = smem + GEMM_STAGES * MT * GEMM_A_BYTES;      // [S][16 KB]
    GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(b_stages + GEMM_STAGES * GEMM_B_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * GEMM_BN;
    const int m0 = blockIdx.y * (MT * GEMM_BM);
    const int nkb = p.K / GEMM_BK;
    constexpr uint32_t TMEM_COLS = MT * GEMM_BN;  // 128 or 256: a power of two >= 32

    if (tid == 0) {
        for (int s = 0; s < GEMM_STAGES; ++s) {
            mbar_init(&bars->full_a[s], 1);
            mbar_init(&bars->full_b[s], GEMM_DEQ_WARPS);
            mbar_init(&bars->empty[s], 1);
        }
        mbar_init(&bars->tmem_full, 1);
        bars->failed = 0;
        mbar_init_fence();
    }
    if (warp == 2) tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int issued = 0;
            bool ok = true;
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % GEMM_STAGES;
                if (!mbar_wait_bounded(&bars->empty[s], ((kb / GEMM_STAGES) & 1) ^ 1)) {
                    record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, kb);
                    ok = false;
                    break;
                }
                mbar_arrive_expect_tx(&bars->full_a[s], MT * GEMM_A_BYTES);
#pragma unroll
                for (int t = 0; t < MT; ++t)
                    tma_load_2d(a_stages + (size_t)(s * MT + t) * GEMM_A_BYTES, &tmap_x, kb * GEMM_BK, m0 + t * GEMM_BM, &bars->full_a[s]);
                issued = kb + 1;
            }
            if (!ok) {  // let every copy already issued land before the CTA may exit
                for (int kb = max(0, issued - GEMM_STAGES); kb < issued; ++kb)
                    if (!mbar_wait_bounded(&bars->full_a[kb % GEMM_STAGES], (kb / GEMM_STAGES) & 1)) {
                        record_failure(p.status, STATUS_WAIT_DRAIN_TIMEOUT, kb);
                        break;
                    }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(ElemFormat<T>::value, GEMM_BM, GEMM_BN);
            bool ok = true;
            for (int kb = 0; kb < nkb && ok; ++kb) {
                const int s = kb % GEMM_STAGES;
                const uint32_t ph = (kb / GEMM_STAGES) & 1;
                if (!mbar_wait_bounded(&bars->full_a[s], ph) || !mbar_wait_bounded(&bars->full_b[s], ph)) {
                    record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, kb);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint64_t db = make_smem_desc_sw128(smem_u32(b_stages + (size_t)s * GEMM_B_BYTES));
#pragma unroll
                for (int t = 0; t < MT; ++t) {
                    const uint64_t da = make_smem_desc_sw128(smem_u32(a_stages + (size_t)(s * MT + t) * GEMM_A_BYTES));
#pragma unroll
                    for (int k = 0; k < GEMM_BK / 16; ++k)  // 16 k = 32 bytes along the swizzled row: +2 in the address field
                        tc_mma_f16(tmem_base + t * GEMM_BN, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                }
                tc_commit(&bars->empty[s]);  // frees the stage when these MMAs have read it
            }
            if (ok) tc_commit(&bars->tmem_full);
            else bars->failed = 1;
        }
    } else if (warp >= 4) {
        // ---------------- dequantization ----------------
        const int dt = tid - 128;            // 0..255
        const int r = dt & (GEMM_BN - 1);    // weight row of the tile
        const int h = dt >> 7;               // which 32 of the 64 k (warp-uniform)
        const int wrow = n0 + r;
        const bool row_ok = wrow < p.N;
        const uint8_t* rowp = p.w + (size_t)(row_ok ? wrow : 0) * p.row_bytes;
        Dequant<TYPE> cur, nxt;
        bool ok = true;
        if (nkb > 0) cur.load(rowp, 0, h);
        for (int kb = 0; kb < nkb; ++kb) {
            const int s = kb % GEMM_STAGES;
            if (kb + 1 < nkb) nxt.load(rowp, kb + 1, h);  // software prefetch of the next packed unit
            float v[32];
            cur.values(kb, h, v);
            if (!row_ok) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = 0.0f;
            }
            if (ok && !mbar_wait_bounded(&bars->empty[s], ((kb / GEMM_STAGES) & 1) ^ 1)) {
                record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, kb);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);  // keep the warp together
            if (ok) {
                store_unit<T>(smem_u32(b_stages + (size_t)s * GEMM_B_BYTES), r, h, v);
                fence_proxy_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->full_b[s]);
            }
            cur = nxt;
        }
        // ---------------- epilogue ----------------
        const int t = (warp - 4) >> 2;       // sub-tile of this warp
        const int quarter = warp & 3;        // TMEM lanes 32 * quarter .. + 31
        if (t < MT) {
            if (ok && !mbar_wait_bounded(&bars->tmem_full, 0)) {
                record_failure(p.status, STATUS_WAIT_MMA_TIMEOUT, 0);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            tc_fence_after();
            const int row = m0 + t * GEMM_BM + quarter * 32 + lane;
            T* yrow = reinterpret_cast<T*>(p.y) + (size_t)row * p.ldy;
            const bool vec_ok = (reinterpret_cast<uintptr_t>(p.y) % 16 == 0) && ((size_t)p.ldy * sizeof(T) % 16 == 0);
            if (ok) {
#pragma unroll 1
                for (int c = 0; c < GEMM_BN / 32; ++c) {
                    uint32_t acc[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + t * GEMM_BN + c * 32, acc);
                    const int col0 = n0 + c * 32;
                    if (row < p.M) {
                        if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint4 o;
                                o.x = pack2<T>(__uint_as_float(acc[8 * q]), __uint_as_float(acc[8 * q + 1]));
                                o.y = pack2<T>(__uint_as_float(acc[8 * q + 2]), __uint_as_float(acc[8 * q + 3]));
                                o.z = pack2<T>(__uint_as_float(acc[8 * q + 4]), __uint_as_float(acc[8 * q + 5]));
                                o.w = pack2<T>(__uint_as_float(acc[8 * q + 6]), __uint_as_float(acc[8 * q + 7]));
                                *reinterpret_cast<uint4*>(yrow + col0 + 8 * q) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < p.N) yrow[col0 + j] = from_float<T>(__uint_as_float(acc[j]));
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---------------------------------------------------------------------------------------------
// Second kernel: the same tile GEMM, but the packed weight rows first come into shared memory with asynchronous copies,
// 256 k of every row of the tile at a time, and the dequantization warps read them from there. One row per lane in
// global memory meant scattered 4-byte loads for the 2-byte-aligned Q6_K / Q8_0 blocks; here every global access is
// a 144 .. 272 byte contiguous copy. Needs K a multiple of 256 and rows that start on 16-byte boundaries.
//   warp 3    issues the packed-row copies (16-byte cp.async pieces, 256 k of every row per chunk)
// The chunk of a row lands at raw + r * PITCH (PITCH an odd multiple of 16 bytes: conflict-free 128-bit reads with
// one row per lane); for Q6_K the copy starts at the 16-byte boundary below the superblock, which then begins `o`
// bytes into the slot with o = (210 * chunk) & 15 the same for every row.
// ---------------------------------------------------------------------------------------------
constexpr int GEMM2_STAGES = 3;
constexpr int GEMM2_RAW_STAGES = 2;

template <int TYPE> struct RawChunk;
template <> struct RawChunk<TYPE_Q4_K> { static constexpr int BYTES = 144, COPY = 144, PITCH = 144; };
template <> struct RawChunk<TYPE_Q6_K> { static constexpr int BYTES = 210, COPY = 224, PITCH = 240; };
template <> struct RawChunk<TYPE_Q8_0> { static constexpr int BYTES = 272, COPY = 272, PITCH = 272; };

struct Gemm2Barriers {
    uint64_t full_a[GEMM2_STAGES];
    uint64_t full_b[GEMM2_STAGES];
    uint64_t empty[GEMM2_STAGES];
    uint64_t raw_full[GEMM2_RAW_STAGES];
    uint64_t raw_empty[GEMM2_RAW_STAGES];
    uint64_t tmem_full[2], tmem_empty[2];
    uint32_t tmem_base;
};

// 32 values of unit (k block j of the chunk, half h) of the row whose chunk starts at shared address `rb`
template <int TYPE> struct RawDequant;

template <> struct RawDequant<TYPE_Q4_K> {
    template <int J>
    static __device__ __forceinline__ void values(uint32_t rb, int, int h, float (&v)[32]) {
        const uint4 hdr = lds128(rb);
        const uint4 q0 = lds128(rb + 16 + 32 * J), q1 = lds128(rb + 32 + 32 * J);
        const int j = 2 * J + h;  // sub-block
        uint32_t sc, m;
        if (j < 4) {
            sc = (hdr.y >> (8 * j)) & 0x3fu;
            m = (hdr.z >> (8 * j)) & 0x3fu;
        } else {
            const int jj = j - 4;
            const uint32_t lo = (hdr.w >> (8 * jj)) & 0xffu;
            sc = (lo & 0xfu) | ((((hdr.y >> (8 * jj)) & 0xffu) >> 6) << 4);
            m = (lo >> 4) | ((((hdr.z >> (8 * jj)) & 0xffu) >> 6) << 4);
        }
        const float dl = half_bits_to_float(hdr.x) * byte_to_float(sc);
        const float ml = half_bits_to_float(hdr.x >> 16) * byte_to_float(m);
        const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const int sh = 4 * h;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t nib = (w[i] >> sh) & 0x0f0f0f0fu;
            v[4 * i + 0] = fmaf(dl, byte_as_magic<0>(nib) - 8388608.0f, -ml);
            v[4 * i + 1] = fmaf(dl, byte_as_magic<1>(nib) - 8388608.0f, -ml);
            v[4 * i + 2] = fmaf(dl, byte_as_magic<2>(nib) - 8388608.0f, -ml);
            v[4 * i + 3] = fmaf(dl, byte_as_magic<3>(nib) - 8388608.0f, -ml);
        }
    }
};

template <> struct RawDequant<TYPE_Q8_0> {
    // block b = 2J + h of the eight in the chunk starts at byte 34 b: f16 d, 32 int8
    template <int OFF>
    static __device__ __forceinline__ void block(uint32_t rb, float (&v)[32]) {
        constexpr int A = OFF & ~15, O = OFF & 15;
        uint32_t c[12], w[9];
        lds_chunks<3>(rb + A, c);
        extract_words<O, 9>(c, w);  // bytes OFF .. OFF + 35
        const float d = half_bits_to_float(w[0]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t q = __funnelshift_r(w[i], w[i + 1], 16) ^ 0x80808080u;
            v[4 * i + 0] = d * (byte_as_magic<0>(q) - 8388736.0f);
            v[4 * i + 1] = d * (byte_as_magic<1>(q) - 8388736.0f);
            v[4 * i + 2] = d * (byte_as_magic<2>(q) - 8388736.0f);
            v[4 * i + 3] = d * (byte_as_magic<3>(q) - 8388736.0f);
        }
    }
    template <int J>
    static __device__ __forceinline__ void values(uint32_t rb, int, int h, float (&v)[32]) {
        if (h == 0) block<34 * (2 * J)>(rb, v);
        else block<34 * (2 * J + 1)>(rb, v);
    }
};

template <> struct RawDequant<TYPE_Q6_K> {
    // O = where the superblock starts inside the 16-byte-aligned slot; every field offset used below is a multiple of 16,
    // so all of them share that misalignment
    template <int O>
    static __device__ __forceinline__ void unit(uint32_t rb, int J, int h, float (&v)[32]) {
        const int n = J >> 1, p = J & 1, qd = 2 * p + h;
        uint32_t cl[12], ch[12], ql[8], qh[8];
        lds_chunks<3>(rb + 64 * n + 32 * h, cl);   // bytes O .. O+31 of this window hold ql[64n + 32h ..]
        lds_chunks<3>(rb + 128 + 32 * n, ch);      // qh[32n ..]
        extract_words<O, 8>(cl, ql);
        extract_words<O, 8>(ch, qh);
        const uint32_t sc2 = lds16(rb + O + 192 + 8 * n + 2 * qd);
        const float d = half_bits_to_float(lds16(rb + O + 208));
        const float s0 = d * (float)(int)(int8_t)(sc2 & 0xffu), s1 = d * (float)(int)(int8_t)(sc2 >> 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t q4 = ((ql[i] >> (4 * p)) & 0x0f0f0f0fu) | (((qh[i] >> (2 * qd)) & 0x03030303u) << 4);
            const float sc = i < 4 ? s0 : s1;
            v[4 * i + 0] = sc * (byte_as_magic<0>(q4) - 8388640.0f);
            v[4 * i + 1] = sc * (byte_as_magic<1>(q4) - 8388640.0f);
            v[4 * i + 2] = sc * (byte_as_magic<2>(q4) - 8388640.0f);
            v[4 * i + 3] = sc * (byte_as_magic<3>(q4) - 8388640.0f);
        }
    }
    template <int J>
    static __device__ __forceinline__ void values(uint32_t rb, int kc, int h, float (&v)[32]) {
        switch (kc & 7) {  // (210 * kc) & 15 = 2 * (kc & 7)
            case 0: unit<0>(rb, J, h, v); break;
            case 1: unit<2>(rb, J, h, v); break;
            case 2: unit<4>(rb, J, h, v); break;
            case 3: unit<6>(rb, J, h, v); break;
            case 4: unit<8>(rb, J, h, v); break;
            case 5: unit<10>(rb, J, h, v); break;
            case 6: unit<12>(rb, J, h, v); break;
            default: unit<14>(rb, J, h, v); break;
        }
    }
};

// Persistent: a CTA walks the tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (tile index = weight tile fastest, so the
// CTAs running at one time share activation tiles through L2). The accumulators are double-buffered in TMEM and drained by
// warps of their own, so the epilogue of a tile and the pipeline fill of the next overlap the MMAs.
//   warp 0  TMA producer of the activations       warps 4-11           dequantization
//   warp 1  tcgen05.mma issuer                    warps 12-(11 + 4 MT) epilogue
//   warp 2  TMEM allocation                       warp 3               packed-row copies
//   AQ: warps (12 + 4 MT) .. (11 + 8 MT) expand quantized activations (d * q from the reference's 144-byte blocks) into
//   the A stages instead of warp 0's TMA loads; OutT is the output type (the operands stay 16-bit).
template <int MT, bool AQ = false> constexpr int gemm2_threads() { return 32 * (4 + GEMM_DEQ_WARPS + 4 * MT + (AQ ? 4 * MT : 0)); }

// 32 accumulator columns of one token row -> global memory in OutT
template <typename OutT>
__device__ __forceinline__ void store_row32(OutT* yrow, int col0, int N, bool vec_ok, const uint32_t (&acc)[32]) {
    if (vec_ok && col0 + 32 <= N) {
        if constexpr (sizeof(OutT) == 4) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4*>(yrow + col0 + 4 * q) = make_uint4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 o;
                o.x = pack2<OutT>(__uint_as_float(acc[8 * q]), __uint_as_float(acc[8 * q + 1]));
                o.y = pack2<OutT>(__uint_as_float(acc[8 * q + 2]), __uint_as_float(acc[8 * q + 3]));
                o.z = pack2<OutT>(__uint_as_float(acc[8 * q + 4]), __uint_as_float(acc[8 * q + 5]));
                o.w = pack2<OutT>(__uint_as_float(acc[8 * q + 6]), __uint_as_float(acc[8 * q + 7]));
                *reinterpret_cast<uint4*>(yrow + col0 + 8 * q) = o;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (col0 + j < N) yrow[col0 + j] = from_float<OutT>(__uint_as_float(acc[j]));
    }
}

template <int TYPE, typename T, int MT, bool AQ = false, typename OutT = T>
__global__ void __launch_bounds__(gemm2_threads<MT, AQ>(), 1) gemm_tcgen05_staged_kernel(const __grid_constant__ CUtensorMap tmap_x, const GemmParams p) {
    using RC = RawChunk<TYPE>;
    constexpr int RAW_BYTES = GEMM_BN * RC::PITCH + 64;  // + slack: reads may run a few bytes past the last row's slot
    extern __shared__ uint8_t gemm_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(gemm_smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* a_stages = smem;                                         // [S][MT][16 KB]
    uint8_t* b_stages = smem + GEMM2_STAGES * MT * GEMM_A_BYTES;      // [S][16 KB]
    uint8_t* raw_stages = b_stages + GEMM2_STAGES * GEMM_B_BYTES;     // [2][RAW_BYTES rounded to 128]
    constexpr int RAW_STRIDE = (RAW_BYTES + 127) & ~127;
    Gemm2Barriers* bars = reinterpret_cast<Gemm2Barriers*>(raw_stages + GEMM2_RAW_STAGES * RAW_STRIDE);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkb = p.K / GEMM_BK;
    const int nkc = p.K / 256;
    const int nx = (p.N + GEMM_BN - 1) / GEMM_BN;
    const int ntiles = nx * ((p.M + MT * GEMM_BM - 1) / (MT * GEMM_BM));
    constexpr uint32_t BUF_COLS = MT * GEMM_BN;
    constexpr uint32_t TMEM_COLS = 2 * BUF_COLS;

    if (tid == 0) {
        for (int s = 0; s < GEMM2_STAGES; ++s) {
            mbar_init(&bars->full_a[s], AQ ? 4 * MT : 1);
            mbar_init(&bars->full_b[s], GEMM_DEQ_WARPS);
            mbar_init(&bars->empty[s], 1);
        }
        for (int s = 0; s < GEMM2_RAW_STAGES; ++s) {
            mbar_init(&bars->raw_full[s], 32);  // one arrival per lane of the packed-row producer warp
            mbar_init(&bars->raw_empty[s], GEMM_DEQ_WARPS);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->tmem_full[s], 1);
            mbar_init(&bars->tmem_empty[s], 4 * MT);
        }
        mbar_init_fence();
    }
    if (warp == 2) tmem_alloc(&bars->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&bars->tmem_base);

    if (warp == 0) {
        // ---------------- TMA producer of the activations ----------------
        if (lane == 0 && !AQ) {
            int kbg = 0;  // k-blocks issued so far, over all tiles
            bool ok = true;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
                const int m0 = (tile / nx) * (MT * GEMM_BM);
                for (int kb = 0; kb < nkb; ++kb, ++kbg) {
                    const int s = kbg % GEMM2_STAGES;
                    if (!mbar_wait_bounded(&bars->empty[s], ((kbg / GEMM2_STAGES) & 1) ^ 1)) {
                        record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, kbg);
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&bars->full_a[s], MT * GEMM_A_BYTES);
#pragma unroll
                    for (int t = 0; t < MT; ++t)
                        tma_load_2d(a_stages + (size_t)(s * MT + t) * GEMM_A_BYTES, &tmap_x, kb * GEMM_BK, m0 + t * GEMM_BM, &bars->full_a[s]);
                }
            }
            if (!ok) {  // let every copy already issued land before the CTA may exit
                for (int q = max(0, kbg - GEMM2_STAGES); q < kbg; ++q)
                    if (!mbar_wait_bounded(&bars->full_a[q % GEMM2_STAGES], (q / GEMM2_STAGES) & 1)) {
                        record_failure(p.status, STATUS_WAIT_DRAIN_TIMEOUT, q);
                        break;
                    }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_f16(ElemFormat<T>::value, GEMM_BM, GEMM_BN);
            bool ok = true;
            const uint64_t da0 = make_smem_desc_sw128(smem_u32(a_stages));
            const uint64_t db0 = make_smem_desc_sw128(smem_u32(b_stages));
            int s = 0;
            uint32_t ph = 0;
            bool ready = false;  // the polls made while the previous block's MMAs were issued found this block complete
            int ti = 0;
            for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x, ++ti) {
                const int buf = ti & 1;
                if (!mbar_wait_bounded(&bars->tmem_empty[buf], ((ti >> 1) & 1) ^ 1)) {  // the epilogue has drained this buffer
                    record_failure(p.status, STATUS_WAIT_MMA_TIMEOUT, 2000 + ti);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d0 = tmem_base + buf * BUF_COLS;
                for (int kb = 0; kb < nkb; ++kb) {
                    // both barriers polled together: a poll's round trip through the busy shared-memory pipe costs
                    // hundreds of cycles, more than the tensor core needs for a block, so they must not add up
                    if (!ready && !mbar_wait2_bounded(&bars->full_a[s], ph, &bars->full_b[s], ph)) {
                        record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, kb);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t db = db0 + (uint64_t)(s * (GEMM_B_BYTES >> 4));
                    const uint64_t da = da0 + (uint64_t)(s * MT * (GEMM_A_BYTES >> 4));
                    const int cur = s;
                    if (++s == GEMM2_STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                    // the next block's barriers (of this tile or the next): their answers come back during the issue
                    bool n0 = false, n1 = false;
                    if (kb + 1 < nkb || tile + (int)gridDim.x < ntiles) {  // not after the very last block: nothing would ever arrive
                        n0 = mbar_try_wait(&bars->full_a[s], ph);
                        n1 = mbar_try_wait(&bars->full_b[s], ph);
                    }
#pragma unroll
                    for (int t = 0; t < MT; ++t) {
#pragma unroll
                        for (int k = 0; k < GEMM_BK / 16; ++k)
                            tc_mma_f16(d0 + t * GEMM_BN, da + (uint64_t)(t * (GEMM_A_BYTES >> 4) + 2 * k), db + 2 * k, idesc,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    tc_commit(&bars->empty[cur]);
                    ready = n0 && n1;
                }
                if (ok) tc_commit(&bars->tmem_full[buf]);
            }
        }
    } else if (warp == 3) {
        // ---------------- packed-row producer: 256 k of every row of the tile per chunk ----------------
        bool ok = true;
        int kcg = 0;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            const int n0 = (tile % nx) * GEMM_BN;
            const int rows_valid = min(GEMM_BN, p.N - n0);
            for (int kc = 0; kc < nkc; ++kc, ++kcg) {
                const int rs = kcg % GEMM2_RAW_STAGES;
                if (!mbar_wait_bounded(&bars->raw_empty[rs], ((kcg / GEMM2_RAW_STAGES) & 1) ^ 1)) {
                    if (lane == 0) record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, 1000 + kcg);
                    ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // 16-byte asynchronous copies, consecutive lanes on consecutive pieces of a row (a bulk copy per row would
                // cost the TMA unit more per copy than these small rows are worth); each lane's copies signal the barrier
                uint8_t* stage = raw_stages + (size_t)rs * RAW_STRIDE;
                constexpr int PIECES = RC::COPY / 16;
                const int total = rows_valid * PIECES;
                for (int idx = lane; idx < total; idx += 32) {
                    const int r = idx / PIECES, piece = idx - r * PIECES;
                    const uint8_t* src = p.w + (size_t)(n0 + r) * p.row_bytes + (size_t)kc * RC::BYTES;
                    src = reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(src) & ~(uintptr_t)15) + 16 * piece;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(stage + (size_t)r * RC::PITCH + 16 * piece)), "l"(src) : "memory");
                }
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars->raw_full[rs])) : "memory");
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");  // nothing of this warp may still be writing when the CTA exits
    } else if (warp >= 4 && warp < 4 + GEMM_DEQ_WARPS) {
        // ---------------- dequantization from the staged packed rows ----------------
        const int dt = tid - 128;
        const int r = dt & (GEMM_BN - 1);
        const int h = dt >> 7;
        bool ok = true;
        int kcg = 0;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            const int n0 = (tile % nx) * GEMM_BN;
            const bool row_ok = r < min(GEMM_BN, p.N - n0);
            for (int kc = 0; kc < nkc; ++kc, ++kcg) {
                const int rs = kcg % GEMM2_RAW_STAGES;
                if (ok && !mbar_wait_bounded(&bars->raw_full[rs], (kcg / GEMM2_RAW_STAGES) & 1)) {
                    record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, 1000 + kcg);
                    ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t rb = smem_u32(raw_stages + (size_t)rs * RAW_STRIDE) + (uint32_t)r * RC::PITCH;
#pragma unroll
                for (int J = 0; J < 4; ++J) {
                    const int kbg = 4 * kcg + J;  // every tile has 4 nkc k-blocks, so this also counts over tiles
                    const int s = kbg % GEMM2_STAGES;
                    float v[32];
                    // polled before the arithmetic so that the poll's round trip overlaps it
                    const bool free_now = mbar_try_wait(&bars->empty[s], ((kbg / GEMM2_STAGES) & 1) ^ 1);
                    if (row_ok) {
                        if (J == 0) RawDequant<TYPE>::template values<0>(rb, kc, h, v);
                        else if (J == 1) RawDequant<TYPE>::template values<1>(rb, kc, h, v);
                        else if (J == 2) RawDequant<TYPE>::template values<2>(rb, kc, h, v);
                        else RawDequant<TYPE>::template values<3>(rb, kc, h, v);
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = 0.0f;
                    }
                    if (!free_now && !mbar_wait_bounded(&bars->empty[s], ((kbg / GEMM2_STAGES) & 1) ^ 1)) {
                        record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, kbg);
                        ok = false;
                    }
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    store_unit<T>(smem_u32(b_stages + (size_t)s * GEMM_B_BYTES), r, h, v);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->full_b[s]);
                }
                if (!ok) break;
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->raw_empty[rs]);  // this warp has read the chunk
            }
        }
    } else if (warp >= 4 + GEMM_DEQ_WARPS && warp < 4 + GEMM_DEQ_WARPS + 4 * MT) {
        // ---------------- epilogue: one warp per 32 token rows of a sub-tile ----------------
        const int e = warp - (4 + GEMM_DEQ_WARPS);
        const int t = e >> 2;
        const int quarter = warp & 3;  // the TMEM lanes a warp may read: 32 * (warp % 4)
        const bool vec_ok = (reinterpret_cast<uintptr_t>(p.y) % 16 == 0) && ((size_t)p.ldy * sizeof(OutT) % 16 == 0);
        bool ok = true;
        int ti = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++ti) {
            const int buf = ti & 1;
            const int n0 = (tile % nx) * GEMM_BN;
            const int m0 = (tile / nx) * (MT * GEMM_BM);
            if (!mbar_wait_bounded(&bars->tmem_full[buf], (ti >> 1) & 1)) {
                record_failure(p.status, STATUS_WAIT_MMA_TIMEOUT, ti);
                ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int row = m0 + t * GEMM_BM + quarter * 32 + lane;
            OutT* yrow = reinterpret_cast<OutT*>(p.y) + (size_t)row * p.ldy;
#pragma unroll 1
            for (int c = 0; c < GEMM_BN / 32; ++c) {
                uint32_t acc[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BUF_COLS + t * GEMM_BN + c * 32, acc);
                if (row < p.M) store_row32<OutT>(yrow, n0 + c * 32, p.N, vec_ok, acc);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tmem_empty[buf]);  // the accumulators are in registers or stored: reuse the buffer
        }
    } else if (AQ && warp >= 4 + GEMM_DEQ_WARPS + 4 * MT) {
        // ---------------- quantized activations -> A stages: thread = token row of the tile, both 32-k halves of a k-block.
        // d * q is formed in f32 and rounded once to the operand type, as the dequantized weights are. ----------------
        const int c = tid - 32 * (4 + GEMM_DEQ_WARPS + 4 * MT);
        const int t = c >> 7, r = c & (GEMM_BM - 1);
        bool ok = true;
        int kbg = 0;
        for (int tile = blockIdx.x; tile < ntiles && ok; tile += gridDim.x) {
            const int m0 = (tile / nx) * (MT * GEMM_BM);
            const int token = m0 + t * GEMM_BM + r;
            const bool token_ok = token < p.M;
            for (int kb = 0; kb < nkb; ++kb, ++kbg) {
                const int s = kbg % GEMM2_STAGES;
                // the block of 128 k this k-block lies in; loads go out before the wait for the stage
                const uint8_t* blk = p.aq + ((size_t)(kb >> 1) * p.M + (token_ok ? token : 0)) * MMQ_BLOCK_BYTES;
                const uint4 sc = __ldg(reinterpret_cast<const uint4*>(blk));
                uint4 qv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) qv[i] = __ldg(reinterpret_cast<const uint4*>(blk + 16 + 64 * (kb & 1)) + i);
                const bool free_now = mbar_try_wait(&bars->empty[s], ((kbg / GEMM2_STAGES) & 1) ^ 1);
                if (!free_now && !mbar_wait_bounded(&bars->empty[s], ((kbg / GEMM2_STAGES) & 1) ^ 1)) {
                    record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, 5000 + kbg);
                    ok = false;
                }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
                const uint32_t a_addr = smem_u32(a_stages + (size_t)(s * MT + t) * GEMM_A_BYTES);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const uint32_t sw = scw[2 * (kb & 1) + h];
                    const float d = token_ok ? (p.aq_ds4 ? half_bits_to_float(sw) : __uint_as_float(sw)) : 0.0f;
                    const uint32_t w8[8] = {qv[2 * h].x, qv[2 * h].y, qv[2 * h].z, qv[2 * h].w, qv[2 * h + 1].x, qv[2 * h + 1].y, qv[2 * h + 1].z, qv[2 * h + 1].w};
                    float v[32];
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint32_t u = w8[i] ^ 0x80808080u;  // q + 128 as unsigned bytes
                        v[4 * i + 0] = d * (byte_as_magic<0>(u) - 8388736.0f);  // 2^23 + 128
                        v[4 * i + 1] = d * (byte_as_magic<1>(u) - 8388736.0f);
                        v[4 * i + 2] = d * (byte_as_magic<2>(u) - 8388736.0f);
                        v[4 * i + 3] = d * (byte_as_magic<3>(u) - 8388736.0f);
                    }
                    store_unit<T>(a_addr, r, h, v);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars->full_a[s]);
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 2) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Prefill matmul on quantized activations for shapes the tile kernel does not take (K not a multiple of 256, packed
// rows that are not a multiple of 16 bytes, unaligned weights): a warp per weight row and 8 tokens, 32-value blocks over
// the lanes, integer dot products per block with the block scales applied in f32 - the reference MMQ's arithmetic.
template <int TYPE, typename OutT>
__global__ void __launch_bounds__(256) mmq_simple_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ aq, OutT* __restrict__ y,
                                                         int M, int N, int K, int ldy, int row_bytes, int ds4) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int tok0 = blockIdx.y * 8;
    if (row >= N) return;
    const uint8_t* rp = w + (size_t)row * row_bytes;
    float acc[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) acc[t] = 0.0f;
    for (int kb = lane; kb < K / 32; kb += 32) {
        int wq[32];
        float s0 = 0.0f, s1 = 0.0f, mn = 0.0f;  // Q4_K: s0 = d sc, mn = dmin m; Q6_K: s0, s1 = d sc of the two halves; Q8_0: s0 = d
        if (TYPE == TYPE_Q8_0) {
            const uint8_t* b = rp + (size_t)kb * Q8_0_BYTES;
            s0 = half_bits_to_float((uint32_t)b[0] | ((uint32_t)b[1] << 8));
            for (int l = 0; l < 32; ++l) wq[l] = (int)(int8_t)b[2 + l];
        } else if (TYPE == TYPE_Q4_K) {
            const int j = kb & 7;
            const uint8_t* sb = rp + (size_t)(kb >> 3) * Q4_K_BYTES;
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
            const uint8_t* sb = rp + (size_t)(kb >> 3) * Q6_K_BYTES;
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
        for (int t = 0; t < 8; ++t) {
            const int token = tok0 + t;
            if (token >= M) break;
            const uint8_t* blk = aq + ((size_t)(kb >> 2) * M + token) * MMQ_BLOCK_BYTES;
            const int8_t* aqv = reinterpret_cast<const int8_t*>(blk + 16 + 32 * (kb & 3));
            const float xd = ds4 ? half_bits_to_float(reinterpret_cast<const uint32_t*>(blk)[kb & 3]) : reinterpret_cast<const float*>(blk)[kb & 3];
            int d0 = 0, d1 = 0, sum = 0;
            for (int l = 0; l < 16; ++l) { d0 += wq[l] * (int)aqv[l]; sum += (int)aqv[l]; }
            for (int l = 16; l < 32; ++l) { d1 += wq[l] * (int)aqv[l]; sum += (int)aqv[l]; }
            if (TYPE == TYPE_Q6_K) acc[t] += xd * (s0 * (float)d0 + s1 * (float)d1);
            else if (TYPE == TYPE_Q4_K) acc[t] += s0 * (xd * (float)(d0 + d1)) - mn * (xd * (float)sum);
            else acc[t] += s0 * (xd * (float)(d0 + d1));
        }
    }
    for (int t = 0; t < 8; ++t) {
        const float v = warp_sum(acc[t]);
        if (lane == 0 && tok0 + t < M) y[(size_t)(tok0 + t) * ldy + row] = from_float<OutT>(v);
    }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------
template <int TYPE, typename T, int MT, bool AQ = false, typename OutT = T>
static int launch_gemm_staged_mt(const CUtensorMap& map, const GemmParams& p, cudaStream_t s) {
    auto kernel = gemm_tcgen05_staged_kernel<TYPE, T, MT, AQ, OutT>;
    constexpr int RAW_STRIDE = ((GEMM_BN * RawChunk<TYPE>::PITCH + 64) + 127) & ~127;
    const size_t smem = 1024 + (size_t)GEMM2_STAGES * (MT * GEMM_A_BYTES + GEMM_B_BYTES) + (size_t)GEMM2_RAW_STAGES * RAW_STRIDE +
                        sizeof(Gemm2Barriers);
    static PerDeviceOnce configured;  // per instantiation and device
    const cudaError_t attr_err =
        configured.run([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
    if (attr_err != cudaSuccess) return (int)attr_err;
    const int ntiles = ((p.N + GEMM_BN - 1) / GEMM_BN) * ((p.M + MT * GEMM_BM - 1) / (MT * GEMM_BM));
    const int sms = runtime_info().sm_count;
    kernel<<<ntiles < sms ? ntiles : sms, gemm2_threads<MT, AQ>(), smem, s>>>(map, p);
    return (int)cudaGetLastError();
}

template <int TYPE, typename T, int MT>
static int launch_gemm_mt(const CUtensorMap& map, const GemmParams& p, cudaStream_t s) {
    auto kernel = gemm_tcgen05_kernel<TYPE, T, MT>;
    const size_t smem = 1024 + (size_t)GEMM_STAGES * (MT * GEMM_A_BYTES + GEMM_B_BYTES) + sizeof(GemmBarriers);
    static PerDeviceOnce configured;  // per instantiation and device
    const cudaError_t attr_err =
        configured.run([&] { return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
    if (attr_err != cudaSuccess) return (int)attr_err;
    dim3 grid((unsigned)((p.N + GEMM_BN - 1) / GEMM_BN), (unsigned)((p.M + MT * GEMM_BM - 1) / (MT * GEMM_BM)), 1);
    kernel<<<grid, GEMM_THREADS, smem, s>>>(map, p);
    return (int)cudaGetLastError();
}

template <int TYPE, typename T>
static int launch_gemm_t(const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, cudaStream_t s) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return B200Q_ERR_UNSUPPORTED;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint32_t box[2] = {GEMM_BK, GEMM_BM};
    const CUtensorMapDataType dt = ElemFormat<T>::value == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = encode_tiled_2d_cached(&map, dt, x, dims, (cuuint64_t)ldx * sizeof(T), box, CU_TENSOR_MAP_SWIZZLE_128B,
                                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B);
    if (r != CUDA_SUCCESS) return B200Q_ERR_INVALID;
    GemmParams p{};
    p.w = static_cast<const uint8_t*>(w);
    p.y = y;
    p.M = M;
    p.N = N;
    p.K = K;
    p.ldy = ldy;
    p.row_bytes = K / type_block_elems(TYPE) * type_block_bytes(TYPE);
    p.status = status_ptr();
    // two 128-token sub-tiles per CTA halve the dequantization work per flop; one keeps more CTAs busy on small problems
    const long long tiles2 = (long long)((N + GEMM_BN - 1) / GEMM_BN) * ((M + 2 * GEMM_BM - 1) / (2 * GEMM_BM));
    const bool two = M > GEMM_BM && tiles2 >= runtime_info().sm_count;
    // packed rows staged through shared memory when the layout allows it (whole 256-k chunks, 16-byte aligned rows)
    const bool staged = runtime_info().gemm_direct == 0 && K % 256 == 0 && p.row_bytes % 16 == 0 &&
                        reinterpret_cast<uintptr_t>(w) % 16 == 0;
    if (staged) return two ? launch_gemm_staged_mt<TYPE, T, 2>(map, p, s) : launch_gemm_staged_mt<TYPE, T, 1>(map, p, s);
    return two ? launch_gemm_mt<TYPE, T, 2>(map, p, s) : launch_gemm_mt<TYPE, T, 1>(map, p, s);
}

// The reference's prefill launcher (crates/inference-quant/src/gguf/ffi.rs:911-927, called from fast_mmq.rs:489-512):
// y[token * stride_col_dst + row] = sum_k W[row][k] * (d q)[token][k] with the activations already quantized by
// launch_mmq_quantize_q8_1_{D4,DS4} into 144-byte blocks. The tile kernel expands d * q into its A stages (operands in
// bf16, f32 accumulation); shapes it does not take go to mmq_simple_kernel. tmp_fixup (the reference's stream-k
// scratch) is not needed.
template <int TYPE, typename OutT>
static int launch_mmq_t(const void* w, const void* aq, void* y, long long K, long long N, long long M, long long stride_row_x,
                        long long ldy, int ds4, cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    const int be = type_block_elems(TYPE), bb = type_block_bytes(TYPE);
    if (K <= 0 || K % be != 0 || K > (1LL << 30) || N > (1LL << 30) || M > (1LL << 30) || ldy > (1LL << 30))
        return B200Q_ERR_UNSUPPORTED;
    GemmParams p{};
    p.w = static_cast<const uint8_t*>(w);
    p.y = y;
    p.M = (int)M;
    p.N = (int)N;
    p.K = (int)K;
    p.ldy = (int)ldy;
    p.row_bytes = (int)(stride_row_x * bb);
    p.status = status_ptr();
    p.aq = static_cast<const uint8_t*>(aq);
    p.aq_ds4 = ds4;
    const bool tile_ok = K % 256 == 0 && stride_row_x == K / be && p.row_bytes % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                         reinterpret_cast<uintptr_t>(aq) % 16 == 0;
    if (!tile_ok) {
        if (reinterpret_cast<uintptr_t>(aq) % 4 != 0) return B200Q_ERR_UNSUPPORTED;
        const dim3 grid((unsigned)((N + 7) / 8), (unsigned)((M + 7) / 8), 1);
        mmq_simple_kernel<TYPE, OutT><<<grid, 256, 0, s>>>(p.w, p.aq, static_cast<OutT*>(y), p.M, p.N, p.K, p.ldy, p.row_bytes, ds4);
        return (int)cudaGetLastError();
    }
    CUtensorMap unused_map{};  // the AQ kernels take no tensor map for the activations
    const long long tiles2 = (long long)((N + GEMM_BN - 1) / GEMM_BN) * ((M + 2 * GEMM_BM - 1) / (2 * GEMM_BM));
    const bool two = M > GEMM_BM && tiles2 >= runtime_info().sm_count;
    return two ? launch_gemm_staged_mt<TYPE, __nv_bfloat16, 2, true, OutT>(unused_map, p, s)
               : launch_gemm_staged_mt<TYPE, __nv_bfloat16, 1, true, OutT>(unused_map, p, s);
}

template <int TYPE>
static int launch_mmq(const void* w, const void* aq, void* y, long long K, long long N, long long M, long long stride_row_x, long long ldy,
                      int ds4, int type_dst, cudaStream_t s) {
    // the reference's element codes (crates/inference-quant/src/gguf/fast_mmq.rs:671-676): 0 = f32, 1 = f16, 30 = bf16
    if (type_dst == 0) return launch_mmq_t<TYPE, float>(w, aq, y, K, N, M, stride_row_x, ldy, ds4, s);
    if (type_dst == 1) return launch_mmq_t<TYPE, __half>(w, aq, y, K, N, M, stride_row_x, ldy, ds4, s);
    if (type_dst == 30) return launch_mmq_t<TYPE, __nv_bfloat16>(w, aq, y, K, N, M, stride_row_x, ldy, ds4, s);
    return B200Q_ERR_INVALID;
}

int gemm_dispatch(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, cudaStream_t s) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % GEMM_BK != 0 || K % type_block_elems(type) != 0) return B200Q_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || ((size_t)ldx * 2) % 16 != 0) return B200Q_ERR_UNSUPPORTED;
    if (type == TYPE_Q4_K && reinterpret_cast<uintptr_t>(w) % 16 != 0) return B200Q_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(w) % 2 != 0) return B200Q_ERR_UNSUPPORTED;
#define B200Q_GEMM_CASE(TYPE)                                                                                     \
    if (type == TYPE) {                                                                                           \
        if (elem == ELEM_BF16) return launch_gemm_t<TYPE, __nv_bfloat16>(w, x, y, M, N, K, ldx, ldy, s);          \
        if (elem == ELEM_F16) return launch_gemm_t<TYPE, __half>(w, x, y, M, N, K, ldx, ldy, s);                  \
        return B200Q_ERR_UNSUPPORTED;                                                                             \
    }
    B200Q_GEMM_CASE(TYPE_Q4_K)
    B200Q_GEMM_CASE(TYPE_Q6_K)
    B200Q_GEMM_CASE(TYPE_Q8_0)
#undef B200Q_GEMM_CASE
    return B200Q_ERR_UNSUPPORTED;
}

}  // namespace b200q

// The reference's symbols; void, asynchronous, allocation-free. The activation scale layout follows the weight type as in
// the reference's host (fast_mmq.rs:167-190): Q8_0 and Q6_K blocks carry four f32 d (D4), Q4_K blocks four half2 (d, sum)
// (DS4). cc, nsm, smpbo and warp_size describe the device to the reference's kernel and are not needed here.
#define B200Q_MMQ_LAUNCHER(tag, TYPE, DS4)                                                                                          \
    extern "C" void launch_mmq_gguf_##tag(void* tmp_fixup, const void* x, const void* y, void* dst, int64_t ncols_x, int64_t nrows_x, \
                                          int64_t ncols_y, int64_t stride_row_x, int64_t stride_col_dst, int cc, int nsm,            \
                                          int64_t smpbo, int warp_size, int type_dst, void* stream) {                                \
        (void)tmp_fixup; (void)cc; (void)nsm; (void)smpbo; (void)warp_size;                                                          \
        b200q::note_launch_status(b200q::launch_mmq<TYPE>(x, y, dst, ncols_x, nrows_x, ncols_y, stride_row_x, stride_col_dst, DS4,    \
                                                          type_dst, (cudaStream_t)stream));                                          \
    }
B200Q_MMQ_LAUNCHER(q8_0, b200q::TYPE_Q8_0, 0)
B200Q_MMQ_LAUNCHER(q4_k, b200q::TYPE_Q4_K, 1)
B200Q_MMQ_LAUNCHER(q6_k, b200q::TYPE_Q6_K, 0)
#undef B200Q_MMQ_LAUNCHER

// Decode-time GEMV: dst[b][row] = sum_k W[row][k] * x[b][k] for packed Q8_0 / Q4_K / Q6_K weights in their GGUF
// layout and 1..8 activation rows, replacing the reference's `mmvq_gguf_<type>_<dst>_plain_cuda{1..8}`
// (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:688-759, launcher :1762-1834).
//
// Design (HBM-bound; no tensor cores):
//  * Weight rows are contiguous, so the matrix is one byte stream. Each CTA owns a contiguous range of rows and
//    streams it through a ring of shared-memory stages with 1-D bulk (TMA) copies issued by one producer thread;
//    full/empty mbarriers hand stages to eight consumer warps. Many KB per SM stay in flight with no registers
//    spent on it, and the 2-byte-aligned Q6_K / Q8_0 blocks need no aligned global loads.
//  * Activations are staged once per CTA in shared memory as 80-byte records per 64 values
//    {i8 q[64]; f32 d[2]; f32 d*sum(q)[2]}: the 80-byte stride makes the 128-bit reads conflict-free. They come
//    either from Q8_1 blocks written by the quantize launcher (the reference's two-launch protocol) or straight from
//    bf16/f16/f32 rows (quantized in the prologue with the same formula, one launch).
//  * Consumers unpack nibbles and 6-bit scales in registers, use dp4a on 4 packed int8, fold scales in f32 and
//    reduce with warp shuffles; rows longer than one warp's worth are split across warps and combined through a
//    small shared array in a fixed order, so results are deterministic.
//  * Every mbarrier wait is bounded and reports through the device status word.
#pragma once
#include "common.cuh"
#include "runtime.h"

namespace b200q {

constexpr int GEMV_CONSUMER_WARPS = 8;
constexpr int GEMV_THREADS = (GEMV_CONSUMER_WARPS + 1) * 32;
constexpr int GEMV_MAX_STAGES = 8;
constexpr int ACT_REC_BYTES = 80;  // i8 q[64]; f32 d[2]; f32 ds[2]

enum ActMode : int { ACT_Q8_1 = 0, ACT_RAW_Q8_1 = 1, ACT_RAW_CPU = 2 };

struct GemvParams {
    const uint8_t* w;   // packed weights, row-major blocks, 16-byte aligned, >= 16 readable bytes after the end
    const void* act;    // Q8_1 blocks [B][stride_act] (ACT_Q8_1) or raw rows [B][stride_act elements] (ACT_RAW)
    void* dst;          // [B][stride_dst]
    int K, N;
    int stride_act;
    int stride_dst;
    int row_bytes;
    int rows_per_stage;  // R: rows one stage holds (multiple of row_align and of consumer_warps / warps_per_row)
    int warps_per_row;   // power of two <= 8
    int row_align;       // rows per 16-byte-aligned unit of the byte stream
    int nstages;
    int stage_bytes;     // multiple of 128
    int act_bytes;       // bytes of activation records
    int use_pdl;
    int act_vec;         // raw activations: rows are 16-byte aligned
    unsigned int* status;  // device status word
};

// ---------------------------------------------------------------------------------------------
// Activation staging
// ---------------------------------------------------------------------------------------------

// From Q8_1 blocks: one thread per 32-value block.
template <int B>
__device__ __forceinline__ void stage_acts_q8_1(uint8_t* acts, const uint8_t* vy, int K, int stride_blocks, int tid,
                                                int nthreads) {
    const int nblk = K / 32;
    const int nrec = K / 64;
    for (int i = tid; i < B * nblk; i += nthreads) {
        const int b = i / nblk, kb = i - b * nblk;
        const uint32_t* src = reinterpret_cast<const uint32_t*>(vy + ((size_t)b * stride_blocks + kb) * Q8_1_BYTES);
        uint8_t* rec = acts + ((size_t)b * nrec + (kb >> 1)) * ACT_REC_BYTES;
        const int h = kb & 1;
        const uint32_t ds = src[0];
        int sum = 0;
        uint32_t* qdst = reinterpret_cast<uint32_t*>(rec + 32 * h);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t v = src[1 + j];
            qdst[j] = v;
            sum = dp4a_ss(0x01010101u, v, sum);
        }
        const float d = half_bits_to_float(ds);
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

// From raw rows, quantized here. Each thread takes 8 consecutive values, so 4 lanes share a 32-value block and a warp
// covers 256 values.
//   ACT_RAW_Q8_1: the decode quantizer's arithmetic (d = amax / 127 rounded to f16, q = roundf(x / d)): identical to
//                 running launch_mmvq_gguf_quantize_q8_1_* first.
//   ACT_RAW_CPU:  the reference CPU path's activation format for the weight type: Q8_K for Q4_K / Q6_K (one f32 scale
//                 per 256 values, iscale = -127 / max, crates/inference-tensor/src/quantized/k_quants.rs:2721-2760) and
//                 Q8_0 for Q8_0 (per 32, f16 scale, q = round(x * (1 / d)), quantized/mod.rs:43-56). The integer dot
//                 products then equal the CPU path's exactly.
template <int B, typename src_t, int TYPE, int MODE>
__device__ __forceinline__ void stage_acts_raw(uint8_t* acts, const src_t* x, int K, int stride_elems, bool vec, int tid,
                                               int nthreads) {
    const int chunks = K / 8;
    const int nrec = K / 64;
    const int lane = tid & 31;
    constexpr bool PER_256 = (MODE == ACT_RAW_CPU) && (TYPE != TYPE_Q8_0);
    const unsigned gmask = PER_256 ? 0xffffffffu : (0xFu << (lane & 28));
    for (int i = tid; i < B * chunks; i += nthreads) {
        const int b = i / chunks, c = i - b * chunks;
        float v[8];
        load8<src_t>(x + (size_t)b * stride_elems + 8 * c, vec, v);
        int q[8];
        float d_store, d_used;
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
                d_store = 0.0f;
            } else {
                const float iscale = -127.0f / mx;
#pragma unroll
                for (int j = 0; j < 8; ++j) q[j] = (int)fminf(fmaxf(roundf(iscale * v[j]), -128.0f), 127.0f);
                d_store = 1.0f / iscale;
            }
            d_used = d_store;
        } else {
            float amax = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(v[j]));
            amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(gmask, amax, 2));
            const float d = amax / 127.0f;
            if (MODE == ACT_RAW_CPU) {
                const float id = d != 0.0f ? 1.0f / d : 0.0f;
#pragma unroll
                for (int j = 0; j < 8; ++j) q[j] = (int)roundf(v[j] * id);
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) q[j] = amax == 0.0f ? 0 : (int)roundf(v[j] / d);
            }
            d_store = __half2float(__float2half_rn(d));
            d_used = d_store;
        }
        int sum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) sum += q[j];
        sum += __shfl_xor_sync(gmask, sum, 1);
        sum += __shfl_xor_sync(gmask, sum, 2);
        const uint32_t w0 = (uint32_t)(q[0] & 0xff) | ((uint32_t)(q[1] & 0xff) << 8) | ((uint32_t)(q[2] & 0xff) << 16) |
                            ((uint32_t)(q[3] & 0xff) << 24);
        const uint32_t w1 = (uint32_t)(q[4] & 0xff) | ((uint32_t)(q[5] & 0xff) << 8) | ((uint32_t)(q[6] & 0xff) << 16) |
                            ((uint32_t)(q[7] & 0xff) << 24);
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
// Per-type decoders. `rowp` points at a weight row inside a shared-memory stage; `item` indexes the row's
// work items; acts points at record 0 of activation row 0; nrec = K / 64.
// ---------------------------------------------------------------------------------------------

// Q4_K: 4 items per superblock; item (s, c) is the 64 values of chunk c: 32 bytes of nibbles, low nibbles are
// sub-block 2c, high nibbles sub-block 2c+1. Activation record index == item index.
template <int B>
__device__ __forceinline__ void q4k_item(const uint8_t* rowp, int item, const uint8_t* acts, int nrec, float (&acc)[B]) {
    const int s = item >> 2, c = item & 3;
    const uint8_t* sb = rowp + s * Q4_K_BYTES;
    const uint4 hdr = *reinterpret_cast<const uint4*>(sb);
    const uint4 w0 = *reinterpret_cast<const uint4*>(sb + 16 + 32 * c);
    const uint4 w1 = *reinterpret_cast<const uint4*>(sb + 32 + 32 * c);
    // 6-bit scale / min of sub-blocks 2c, 2c+1 (crates/inference-tensor/src/quantized/utils.rs:119-129)
    const int sh = (c & 1) * 16;
    const uint32_t a1 = hdr.y >> sh, a2 = hdr.z >> sh, a3 = hdr.w >> sh;
    uint32_t scp, mp;
    if (c < 2) {
        scp = a1 & 0x3f3fu;
        mp = a2 & 0x3f3fu;
    } else {
        scp = (a3 & 0x0f0fu) | ((a1 >> 2) & 0x3030u);
        mp = ((a3 >> 4) & 0x0f0fu) | ((a2 >> 2) & 0x3030u);
    }
    const float d = half_bits_to_float(hdr.x), dmin = half_bits_to_float(hdr.x >> 16);
    const float wsc0 = d * (float)(scp & 0xffu);
    const float wsc1 = d * (float)(scp >> 8) * 0.0625f;  // high nibbles are used as 16 * q
    const float wm0 = dmin * (float)(mp & 0xffu);
    const float wm1 = dmin * (float)(mp >> 8);
    const uint32_t wl[8] = {w0.x & 0x0f0f0f0fu, w0.y & 0x0f0f0f0fu, w0.z & 0x0f0f0f0fu, w0.w & 0x0f0f0f0fu,
                            w1.x & 0x0f0f0f0fu, w1.y & 0x0f0f0f0fu, w1.z & 0x0f0f0f0fu, w1.w & 0x0f0f0f0fu};
    const uint32_t wh[8] = {w0.x & 0xf0f0f0f0u, w0.y & 0xf0f0f0f0u, w0.z & 0xf0f0f0f0u, w0.w & 0xf0f0f0f0u,
                            w1.x & 0xf0f0f0f0u, w1.y & 0xf0f0f0f0u, w1.z & 0xf0f0f0f0u, w1.w & 0xf0f0f0f0u};
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const uint8_t* rec = acts + ((size_t)b * nrec + item) * ACT_REC_BYTES;
        const uint4 q0 = *reinterpret_cast<const uint4*>(rec);
        const uint4 q1 = *reinterpret_cast<const uint4*>(rec + 16);
        const uint4 q2 = *reinterpret_cast<const uint4*>(rec + 32);
        const uint4 q3 = *reinterpret_cast<const uint4*>(rec + 48);
        const float4 f = *reinterpret_cast<const float4*>(rec + 64);
        int dl = 0, dh = 0;
        dl = dp4a_us(wl[0], q0.x, dl); dl = dp4a_us(wl[1], q0.y, dl); dl = dp4a_us(wl[2], q0.z, dl); dl = dp4a_us(wl[3], q0.w, dl);
        dl = dp4a_us(wl[4], q1.x, dl); dl = dp4a_us(wl[5], q1.y, dl); dl = dp4a_us(wl[6], q1.z, dl); dl = dp4a_us(wl[7], q1.w, dl);
        dh = dp4a_us(wh[0], q2.x, dh); dh = dp4a_us(wh[1], q2.y, dh); dh = dp4a_us(wh[2], q2.z, dh); dh = dp4a_us(wh[3], q2.w, dh);
        dh = dp4a_us(wh[4], q3.x, dh); dh = dp4a_us(wh[5], q3.y, dh); dh = dp4a_us(wh[6], q3.z, dh); dh = dp4a_us(wh[7], q3.w, dh);
        acc[b] += wsc0 * (f.x * (float)dl) + wsc1 * (f.y * (float)dh) - (wm0 * f.z + wm1 * f.w);
    }
}
__device__ __forceinline__ int q4k_items(int K) { return K / 64; }

// Reads `N` consecutive 32-bit words starting at the 2-byte-aligned shared address p.
template <int N>
__device__ __forceinline__ void load_words_u16aligned(const uint8_t* p, uint32_t (&out)[N]) {
    const uint32_t addr = smem_u32(p);
    const uint32_t shift = (addr & 2u) * 8u;
    const uint32_t* a = reinterpret_cast<const uint32_t*>(p - (addr & 2u));
    uint32_t prev = a[0];
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const uint32_t next = a[i + 1];
        out[i] = funnel16(prev, next, shift);
        prev = next;
    }
}

// Q6_K: 8 items per superblock; item (s, n, u): half n, bytes l = 8u..8u+7 of that half: 8 values from each of the
// four 32-value quarters (crates/inference-tensor/src/quantized/k_quants.rs:2661-2677). Weights are rebuilt as
// 4 * (q - 32) in a signed byte: ((q ^ 32) << 2) reinterpreted, so no subtraction and one signed dp4a.
template <int B>
__device__ __forceinline__ void q6k_item(const uint8_t* rowp, int item, const uint8_t* acts, int nrec, float (&acc)[B]) {
    const int s = item >> 3, n = (item >> 2) & 1, u = item & 3;
    const uint8_t* sb = rowp + s * Q6_K_BYTES;
    uint32_t qla[2], qlb[2], qh[2], scw[2];
    load_words_u16aligned<2>(sb + 64 * n + 8 * u, qla);        // ql[64n + l]: quarters 0 (low nibble), 2 (high)
    load_words_u16aligned<2>(sb + 64 * n + 32 + 8 * u, qlb);   // ql[64n + 32 + l]: quarters 1, 3
    load_words_u16aligned<2>(sb + 128 + 32 * n + 8 * u, qh);   // qh[32n + l]: 2 bits per quarter
    load_words_u16aligned<2>(sb + 192 + 8 * n, scw);           // scales[8n .. 8n+7]
    const float d = half_bits_to_float(*reinterpret_cast<const unsigned short*>(sb + 208)) * 0.25f;
    // scale of quarter qd, 16-group u/2: scales[8n + 2*qd + (u >> 1)]
    const int sbyte = (u >> 1);
    float wsc[4];
#pragma unroll
    for (int qd = 0; qd < 4; ++qd) {
        const int idx = 2 * qd + sbyte;  // 0..7
        const uint32_t word = idx < 4 ? scw[0] : scw[1];
        const int sc = (int)(int8_t)((word >> (8 * (idx & 3))) & 0xffu);
        wsc[qd] = d * (float)sc;
    }
    uint32_t wq[4][2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const uint32_t la = qla[t], lb = qlb[t], h = qh[t];
        wq[0][t] = ((la << 2) & 0x3c3c3c3cu) | (((h << 6) & 0xc0c0c0c0u) ^ 0x80808080u);
        wq[1][t] = ((lb << 2) & 0x3c3c3c3cu) | (((h << 4) & 0xc0c0c0c0u) ^ 0x80808080u);
        wq[2][t] = ((la >> 2) & 0x3c3c3c3cu) | (((h << 2) & 0xc0c0c0c0u) ^ 0x80808080u);
        wq[3][t] = ((lb >> 2) & 0x3c3c3c3cu) | ((h & 0xc0c0c0c0u) ^ 0x80808080u);
    }
    // activations: quarter qd of half n of superblock s is 32-value block 8s + 4n + qd = record 4s + 2n + (qd>>1),
    // half (qd & 1); this item uses its bytes 8u..8u+7
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const uint8_t* rec0 = acts + ((size_t)b * nrec + 4 * s + 2 * n) * ACT_REC_BYTES;
        float part = 0.0f;
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            const uint8_t* rec = rec0 + (qd >> 1) * ACT_REC_BYTES;
            const uint2 q = *reinterpret_cast<const uint2*>(rec + 32 * (qd & 1) + 8 * u);
            const float d8 = reinterpret_cast<const float*>(rec + 64)[qd & 1];
            int dot = dp4a_ss(wq[qd][0], q.x, 0);
            dot = dp4a_ss(wq[qd][1], q.y, dot);
            part += wsc[qd] * (d8 * (float)dot);
        }
        acc[b] += part;
    }
}
__device__ __forceinline__ int q6k_items(int K) { return K / 32; }

// Q8_0: one item per 64 values = two 34-byte blocks; activation record index == item index.
template <int B>
__device__ __forceinline__ void q80_item(const uint8_t* rowp, int item, const uint8_t* acts, int nrec, float (&acc)[B]) {
    const uint8_t* blk = rowp + item * (2 * Q8_0_BYTES);
    uint32_t w[17];
    load_words_u16aligned<17>(blk, w);  // 68 bytes: d0 q0[32] d1 q1[32]
    // block 0: d in the low half of w[0], qs = bytes 2..33; block 1: d at byte 34 (high half of w[8]), qs bytes 36..67
    const float d0 = half_bits_to_float(w[0]);
    const float d1 = half_bits_to_float(w[8] >> 16);
    uint32_t qa[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) qa[j] = __funnelshift_r(w[j], w[j + 1], 16);
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const uint8_t* rec = acts + ((size_t)b * nrec + item) * ACT_REC_BYTES;
        const uint4 q0 = *reinterpret_cast<const uint4*>(rec);
        const uint4 q1 = *reinterpret_cast<const uint4*>(rec + 16);
        const uint4 q2 = *reinterpret_cast<const uint4*>(rec + 32);
        const uint4 q3 = *reinterpret_cast<const uint4*>(rec + 48);
        const float4 f = *reinterpret_cast<const float4*>(rec + 64);
        int da = 0, db = 0;
        da = dp4a_ss(qa[0], q0.x, da); da = dp4a_ss(qa[1], q0.y, da); da = dp4a_ss(qa[2], q0.z, da); da = dp4a_ss(qa[3], q0.w, da);
        da = dp4a_ss(qa[4], q1.x, da); da = dp4a_ss(qa[5], q1.y, da); da = dp4a_ss(qa[6], q1.z, da); da = dp4a_ss(qa[7], q1.w, da);
        db = dp4a_ss(w[9], q2.x, db); db = dp4a_ss(w[10], q2.y, db); db = dp4a_ss(w[11], q2.z, db); db = dp4a_ss(w[12], q2.w, db);
        db = dp4a_ss(w[13], q3.x, db); db = dp4a_ss(w[14], q3.y, db); db = dp4a_ss(w[15], q3.z, db); db = dp4a_ss(w[16], q3.w, db);
        acc[b] += d0 * (f.x * (float)da) + d1 * (f.y * (float)db);
    }
}
__device__ __forceinline__ int q80_items(int K) { return K / 64; }

template <int TYPE, int B>
__device__ __forceinline__ void decode_item(const uint8_t* rowp, int item, const uint8_t* acts, int nrec, float (&acc)[B]) {
    if (TYPE == TYPE_Q4_K) q4k_item<B>(rowp, item, acts, nrec, acc);
    else if (TYPE == TYPE_Q6_K) q6k_item<B>(rowp, item, acts, nrec, acc);
    else q80_item<B>(rowp, item, acts, nrec, acc);
}
template <int TYPE>
__device__ __forceinline__ int items_per_row(int K) {
    return TYPE == TYPE_Q4_K ? q4k_items(K) : (TYPE == TYPE_Q6_K ? q6k_items(K) : q80_items(K));
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------
template <int TYPE, int B, typename dst_t, int ACT, typename act_t>
__global__ void __launch_bounds__(GEMV_THREADS, 2) gemv_staged_kernel(const GemvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GEMV_MAX_STAGES;
    uint8_t* acts = smem + 128;
    float* partial = reinterpret_cast<float*>(acts + p.act_bytes);                    // [2][R][WPR][B]
    const int partial_floats = p.warps_per_row > 1 ? 2 * p.rows_per_stage * p.warps_per_row * B : 0;
    uint8_t* ring = acts + p.act_bytes + ((partial_floats * 4 + 127) & ~127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = p.nstages, R = p.rows_per_stage, WPR = p.warps_per_row;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        mbar_init_fence();
    }
    __syncthreads();

    // this CTA's rows: a contiguous run of 16-byte-aligned units
    const long long units = (p.N + p.row_align - 1) / p.row_align;
    const int row0 = (int)(units * blockIdx.x / gridDim.x) * p.row_align;
    int row1 = (int)(units * (blockIdx.x + 1) / gridDim.x) * p.row_align;
    if (row1 > p.N) row1 = p.N;
    const int nrows = row1 > row0 ? row1 - row0 : 0;
    const int niter = (nrows + R - 1) / R;

    if (warp == GEMV_CONSUMER_WARPS) {
        // ---------------- producer: one thread streams this CTA's byte range ----------------
        if (lane == 0) {
            bool ok = true;
            int issued = 0;
            for (int it = 0; it < niter && ok; ++it) {
                const int s = it % S;
                if (it >= S) {
                    ok = mbar_wait_bounded(&empty[s], ((it / S) - 1) & 1);
                    if (!ok) { record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, it); break; }
                }
                const int r = row0 + it * R;
                const int rows = min(R, row1 - r);
                const uint32_t bytes = ((uint32_t)rows * (uint32_t)p.row_bytes + 15u) & ~15u;
                mbar_arrive_expect_tx(&full[s], bytes);
                bulk_copy_g2s(ring + (size_t)s * p.stage_bytes, p.w + (size_t)r * p.row_bytes, bytes, &full[s]);
                issued = it + 1;
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
    if (p.use_pdl) grid_dependency_wait();
    if (ACT == ACT_Q8_1)
        stage_acts_q8_1<B>(acts, reinterpret_cast<const uint8_t*>(p.act), p.K, p.stride_act, tid, GEMV_CONSUMER_WARPS * 32);
    else
        stage_acts_raw<B, act_t, TYPE, ACT>(acts, reinterpret_cast<const act_t*>(p.act), p.K, p.stride_act, p.act_vec != 0, tid,
                                            GEMV_CONSUMER_WARPS * 32);
    named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
    if (p.use_pdl) grid_launch_dependents();

    const int nrec = p.K / 64;
    const int items = items_per_row<TYPE>(p.K);
    const int rows_per_pass = GEMV_CONSUMER_WARPS / WPR;
    const int wrow = warp / WPR, wslice = warp % WPR;
    dst_t* dst = reinterpret_cast<dst_t*>(p.dst);
    bool alive = true;

    for (int it = 0; it < niter; ++it) {
        const int s = it % S;
        if (alive && !mbar_wait_bounded(&full[s], (it / S) & 1)) {
            record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, it);
            alive = false;
        }
        // a failed wait is warp-uniform (every lane polls the same barrier); the warp keeps arriving so that
        // the others are not held up, but computes nothing
        const uint8_t* st = ring + (size_t)s * p.stage_bytes;
        const int rbase = row0 + it * R;
        const int rows_here = min(R, row1 - rbase);
        float* part = partial + (size_t)(it & 1) * R * WPR * B;
        for (int pass = 0; pass * rows_per_pass < rows_here; ++pass) {
            const int r_in = pass * rows_per_pass + wrow;
            float acc[B];
#pragma unroll
            for (int b = 0; b < B; ++b) acc[b] = 0.0f;
            if (alive && r_in < rows_here) {
                const uint8_t* rowp = st + (size_t)r_in * p.row_bytes;
                for (int item = wslice * 32 + lane; item < items; item += 32 * WPR)
                    decode_item<TYPE, B>(rowp, item, acts, nrec, acc);
            }
#pragma unroll
            for (int b = 0; b < B; ++b) acc[b] = warp_sum(acc[b]);
            if (lane == 0 && r_in < rows_here) {
                if (WPR == 1) {
#pragma unroll
                    for (int b = 0; b < B; ++b) dst[(size_t)b * p.stride_dst + rbase + r_in] = from_float<dst_t>(acc[b]);
                } else {
#pragma unroll
                    for (int b = 0; b < B; ++b) part[((size_t)r_in * WPR + wslice) * B + b] = acc[b];
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (WPR > 1) {
            named_bar_sync(1, GEMV_CONSUMER_WARPS * 32);
            for (int o = tid; o < rows_here * B; o += GEMV_CONSUMER_WARPS * 32) {
                const int r_in = o / B, b = o - r_in * B;
                float v = 0.0f;
                for (int w = 0; w < WPR; ++w) v += part[((size_t)r_in * WPR + w) * B + b];
                dst[(size_t)b * p.stride_dst + rbase + r_in] = from_float<dst_t>(v);
            }
        }
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
                int dot = 0, s8 = 0;
                for (int l = 0; l < 32; ++l) {
                    const int a = ld_i8(ab + 4 + l);
                    dot += wq[l] * a;
                    s8 += a;
                }
                acc[b] += scale * d8 * (float)dot - minv * d8 * (float)s8;
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
    size_t smem;
};

// Chooses rows per stage, warps per row, ring depth and grid for a shape. `w` is only inspected for alignment
// (nullptr = assume aligned).
static inline GemvPlan plan_gemv(int type, int K, int N, int B, const void* w) {
    const RuntimeInfo& rt = runtime_info();
    GemvPlan plan{};
    GemvParams& p = plan.p;
    const int be = type_block_elems(type), bb = type_block_bytes(type);
    p.K = K;
    p.N = N;
    p.row_bytes = K / be * bb;
    p.row_align = 16 / gcd_int(p.row_bytes, 16);
    p.act_bytes = ((B * (K / 64) * ACT_REC_BYTES) + 127) & ~127;
    p.use_pdl = rt.use_pdl;
    plan.staged = false;
    if (rt.force_simple || K % 64 != 0 || (reinterpret_cast<uintptr_t>(w) & 15) != 0) return plan;

    // rows per stage: ~stage_target bytes, at least one aligned unit; fewer rows than consumer warps means each
    // row is split over several warps
    int rmax = rt.gemv_stage_target / p.row_bytes;
    if (rmax < 1) rmax = 1;
    int R, wpr;
    if (rmax >= GEMV_CONSUMER_WARPS) {
        wpr = 1;
        R = rmax / GEMV_CONSUMER_WARPS * GEMV_CONSUMER_WARPS;
    } else {
        R = 1;
        while (R * 2 <= rmax) R *= 2;
        if (R < p.row_align) R = p.row_align;  // both powers of two <= 8
        wpr = GEMV_CONSUMER_WARPS / R;
    }
    p.rows_per_stage = R;
    p.warps_per_row = wpr;
    p.stage_bytes = (R * p.row_bytes + 16 + 127) & ~127;
    const int partial_bytes = wpr > 1 ? ((2 * R * wpr * B * 4 + 127) & ~127) : 0;
    const int fixed = 128 + p.act_bytes + partial_bytes;
    const int budget = rt.smem_optin - 1024;  // 1 KB per CTA is reserved by the system
    if (budget - fixed < 2 * p.stage_bytes) return plan;  // does not fit: simple kernel
    // two CTAs per SM when each still gets >= 3 stages and >= 48 KB of ring: more warps to hide unpack latency
    int per_cta = budget, ctas_per_sm = 1;
    {
        const int half = rt.smem_per_sm / 2 - 1024;
        const int avail2 = half - fixed;
        if (avail2 >= 3 * p.stage_bytes && avail2 >= 48 * 1024) {
            ctas_per_sm = 2;
            per_cta = half;
        }
    }
    int S = (per_cta - fixed) / p.stage_bytes;
    if (S > GEMV_MAX_STAGES) S = GEMV_MAX_STAGES;
    p.nstages = S;
    plan.smem = (size_t)fixed + (size_t)S * p.stage_bytes;
    const long long units = (N + p.row_align - 1) / p.row_align;
    long long grid = (long long)rt.sm_count * ctas_per_sm;
    if (grid > units) grid = units;
    if (grid < 1) grid = 1;
    plan.grid = (int)grid;
    plan.staged = true;
    return plan;
}

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

template <int TYPE, int B, typename dst_t, int ACT, typename act_t>
static inline int launch_staged(const GemvPlan& plan, cudaStream_t s) {
    auto kernel = gemv_staged_kernel<TYPE, B, dst_t, ACT, act_t>;
    static bool configured = false;  // per instantiation; the attribute is set on the first launch
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             runtime_info().smem_optin - 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    return (int)launch_gemv_kernel(kernel, plan.grid, GEMV_THREADS, plan.smem, s, plan.p.use_pdl != 0, plan.p);
}

template <int TYPE, int B, typename dst_t>
static inline int launch_gemv_b(const void* vx, const void* act, void* dst, int K, int N, int stride_act, int stride_dst,
                                int act_mode, cudaStream_t s) {
    GemvPlan plan = plan_gemv(TYPE, K, N, B, vx);
    plan.p.w = (const uint8_t*)vx;
    plan.p.act = act;
    plan.p.dst = dst;
    plan.p.stride_act = stride_act;
    plan.p.stride_dst = stride_dst;
    plan.p.status = status_ptr();
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
                              int b, int act_mode, cudaStream_t s) {
    if (N <= 0 || K <= 0) return 0;
    switch (b) {
        case 1: return launch_gemv_b<TYPE, 1, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        case 2: return launch_gemv_b<TYPE, 2, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        case 3: return launch_gemv_b<TYPE, 3, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        case 4: return launch_gemv_b<TYPE, 4, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        case 5: return launch_gemv_b<TYPE, 5, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        case 6: return launch_gemv_b<TYPE, 6, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        case 7: return launch_gemv_b<TYPE, 7, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        case 8: return launch_gemv_b<TYPE, 8, dst_t>(vx, act, dst, K, N, stride_act, stride_dst, act_mode, s);
        default: return B200Q_ERR_UNSUPPORTED;
    }
}

// One weight type's dispatcher over the output element type; defined once per type in gemv_<type>.cu.
template <int TYPE>
static inline int gemv_type_dispatch(int dst_elem, const void* vx, const void* act, void* dst, int K, int N, int stride_act,
                                     int stride_dst, int b, int act_mode, cudaStream_t s) {
    if (dst_elem == ELEM_BF16) return launch_gemv<TYPE, __nv_bfloat16>(vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, s);
    if (dst_elem == ELEM_F16) return launch_gemv<TYPE, __half>(vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, s);
    if (dst_elem == ELEM_F32) return launch_gemv<TYPE, float>(vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, s);
    return B200Q_ERR_UNSUPPORTED;
}

}  // namespace b200q

// The reference's launcher symbols for one type (crates/inference-quant/src/gguf/ffi.rs:846-878); stride_col_y is in
// Q8_1 blocks. Launchers return nothing, as the reference's: a failed launch surfaces at the caller's next checked
// CUDA call, and is also kept for b200q_last_launch_status().
#define B200Q_DEFINE_GEMV_TYPE(tag, TYPE)                                                                              \
    namespace b200q {                                                                                                  \
    int gemv_##tag(int dst_elem, const void* vx, const void* act, void* dst, int K, int N, int stride_act,             \
                   int stride_dst, int b, int act_mode, cudaStream_t s) {                                              \
        return note_launch_status(                                                                                     \
            gemv_type_dispatch<TYPE>(dst_elem, vx, act, dst, K, N, stride_act, stride_dst, b, act_mode, s));           \
    }                                                                                                                  \
    }                                                                                                                  \
    extern "C" void launch_mmvq_gguf_##tag##_bf16_plain(const void* vx, const void* vy, void* dst, int ncols_x,        \
                                                        int nrows_x, int stride_col_y, int stride_col_dst, int b_size, \
                                                        void* stream) {                                                \
        b200q::gemv_##tag(b200q::ELEM_BF16, vx, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst, b_size,       \
                          b200q::ACT_Q8_1, (cudaStream_t)stream);                                                      \
    }                                                                                                                  \
    extern "C" void launch_mmvq_gguf_##tag##_f16_plain(const void* vx, const void* vy, void* dst, int ncols_x,         \
                                                       int nrows_x, int stride_col_y, int stride_col_dst, int b_size,  \
                                                       void* stream) {                                                 \
        b200q::gemv_##tag(b200q::ELEM_F16, vx, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst, b_size,        \
                          b200q::ACT_Q8_1, (cudaStream_t)stream);                                                      \
    }                                                                                                                  \
    extern "C" void launch_mmvq_gguf_##tag##_f32_plain(const void* vx, const void* vy, void* dst, int ncols_x,         \
                                                       int nrows_x, int stride_col_y, int stride_col_dst, int b_size,  \
                                                       void* stream) {                                                 \
        b200q::gemv_##tag(b200q::ELEM_F32, vx, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst, b_size,        \
                          b200q::ACT_Q8_1, (cudaStream_t)stream);                                                      \
    }

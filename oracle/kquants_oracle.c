/*
 * CPU oracle for the GGUF quantized-matmul path (Q8_0 / Q4_K / Q6_K weights).
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA kernels are compared with and the
 * timed CPU baseline; nothing on the product path may call it.
 *
 * It restates, in plain C, the arithmetic of the reference's Rust CPU code. The reference cannot be
 * compiled where this runs (it is Rust), so every function names the reference source it follows, by
 * the file's path inside the reference project:
 *   Q  = crates/inference-tensor/src/quantized/k_quants.rs
 *   U  = crates/inference-tensor/src/quantized/utils.rs
 *   M  = crates/inference-tensor/src/quantized/mod.rs
 *   CU = crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_quantize.cu
 *   MQ = crates/inference-quant/kernels/cuda/mmq_gguf/mmq_quantize.cu
 *
 * Pinning: the quantizers are checked against the reference's own known-answer test, FNV-1a-64 hashes
 * of the packed bytes of an LCG-generated 8x512 layer in its `IkLlama` mode
 * (crates/inference-quant/src/gguf/requantize.rs:1071-1152): q8_0, q4_k plain, q6_k plain and q6_k with
 * an importance matrix. The default (`LlamaCpp`) mode shares all code with that mode except where a
 * multiply-add is fused, and has no byte-level pin of its own in the reference: for that mode alone,
 * parity unpinned beyond the shared code, the dequantize round trip and gguf-py's dequantizers.
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fPIC -shared (no -ffast-math: the scale searches are
 * sensitive to contraction and reassociation, U:37-45).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK_K 256
#define QK8_0 32
#define K_SCALE_SIZE 12

enum { ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q6_K = 14 }; /* GGUF type ids, M:582-624 */
enum { ORC_LLAMACPP = 0, ORC_IKLLAMA = 1 };           /* Q:38-44 `Quantizer` */

#pragma pack(push, 1)
typedef struct { uint16_t d; int8_t qs[32]; } block_q8_0;                                 /* Q:150-156 */
typedef struct { uint16_t d; uint16_t s; int8_t qs[32]; } block_q8_1;                     /* Q:158-165 */
typedef struct { uint16_t d; uint16_t dmin; uint8_t scales[12]; uint8_t qs[128]; } block_q4_k; /* Q:188-196 */
typedef struct { uint8_t ql[128]; uint8_t qh[64]; int8_t scales[16]; uint16_t d; } block_q6_k; /* Q:210-218 */
typedef struct { float d; int8_t qs[256]; int16_t bsums[16]; } block_q8_k;                /* Q:220-227 */
#pragma pack(pop)

_Static_assert(sizeof(block_q8_0) == 34, "q8_0");
_Static_assert(sizeof(block_q8_1) == 36, "q8_1");
_Static_assert(sizeof(block_q4_k) == 144, "q4_k");
_Static_assert(sizeof(block_q6_k) == 210, "q6_k");
_Static_assert(sizeof(block_q8_k) == 292, "q8_k");

/* ---------------------------------------------------------------- scalar conversions */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* f32 -> f16, round to nearest even, as the `half` crate's `f16::from_f32` (software path). */
uint16_t orc_f32_to_f16(float value) {
    uint32_t x = f2u(value);
    uint32_t sign = x & 0x80000000u;
    uint32_t exp = x & 0x7F800000u;
    uint32_t man = x & 0x007FFFFFu;
    if (exp == 0x7F800000u) { /* inf / nan */
        uint32_t nan_bit = man == 0 ? 0 : 0x0200u;
        return (uint16_t)((sign >> 16) | 0x7C00u | nan_bit | (man >> 13));
    }
    uint32_t half_sign = sign >> 16;
    int32_t unbiased = (int32_t)(exp >> 23) - 127;
    int32_t half_exp = unbiased + 15;
    if (half_exp >= 0x1F) return (uint16_t)(half_sign | 0x7C00u); /* overflow -> inf */
    if (half_exp <= 0) {                                           /* subnormal or zero */
        if (14 - half_exp > 24) return (uint16_t)half_sign;
        man |= 0x00800000u;
        uint32_t half_man = man >> (14 - half_exp);
        uint32_t round_bit = 1u << (13 - half_exp);
        if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0) half_man += 1;
        return (uint16_t)(half_sign | half_man);
    }
    uint32_t he = (uint32_t)half_exp << 10;
    uint32_t hm = man >> 13;
    uint32_t round_bit = 0x00001000u;
    if ((man & round_bit) != 0 && (man & (3 * round_bit - 1)) != 0)
        return (uint16_t)((half_sign | he | hm) + 1);
    return (uint16_t)(half_sign | he | hm);
}

float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1F;
    uint32_t man = h & 0x3FFu;
    if (exp == 0) {
        if (man == 0) return u2f(sign);
        /* subnormal: value = man * 2^-24 */
        float f = (float)man * 5.9604644775390625e-08f;
        return sign ? -f : f;
    }
    if (exp == 0x1F) return u2f(sign | 0x7F800000u | (man << 13));
    return u2f(sign | ((exp + 112) << 23) | (man << 13));
}

/* f32 -> bf16 round to nearest even, as `half::bf16::from_f32`. */
uint16_t orc_f32_to_bf16(float value) {
    uint32_t x = f2u(value);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x0040u);
    uint32_t round_bit = 0x00008000u;
    if ((x & round_bit) != 0 && (x & (3 * round_bit - 1)) != 0) return (uint16_t)((x >> 16) + 1);
    return (uint16_t)(x >> 16);
}
float orc_bf16_to_f32(uint16_t h) { return u2f((uint32_t)h << 16); }

void orc_widen_bf16(const uint16_t *src, float *dst, int64_t n) { /* M:1417-1434 */
    for (int64_t i = 0; i < n; i++) dst[i] = orc_bf16_to_f32(src[i]);
}
void orc_narrow_bf16(const float *src, uint16_t *dst, int64_t n) { /* M:1436-1453 */
    for (int64_t i = 0; i < n; i++) dst[i] = orc_f32_to_bf16(src[i]);
}
void orc_widen_f16(const uint16_t *src, float *dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = orc_f16_to_f32(src[i]);
}
void orc_narrow_f16(const float *src, uint16_t *dst, int64_t n) {
    for (int64_t i = 0; i < n; i++) dst[i] = orc_f32_to_f16(src[i]);
}

/* Rust's `as i8` on a float saturates. */
static inline int8_t sat_i8(float v) {
    if (v != v) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int8_t)v;
}

/* ---------------------------------------------------------------- rounding helpers (U:3-4, 32-73) */

#define ROUNDING_MAGIC 12582912.0f
#define GROUP_MAX_EPS 1e-15f
#define QKX_FLAT_RANGE 1e-10f

static inline int nearest_int(float v) { /* U:32-35 */
    float r = v + ROUNDING_MAGIC;
    return (int)(f2u(r) & 0x007fffffu) - 0x00400000;
}
static inline float madd(int ik, float a, float b, float c) { /* U:40-45 */
    return ik ? fmaf(a, b, c) : a * b + c;
}
static inline float msub(int ik, float a, float b, float c, float d) { /* U:49-54 */
    return ik ? fmaf(a, b, -(c * d)) : a * b - c * d;
}
static inline int nearest_int_mul(int ik, float a, float b) { /* U:70-73 */
    float r = madd(ik, a, b, ROUNDING_MAGIC);
    return (int)(f2u(r) & 0x007fffffu) - 0x00400000;
}
static inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

/* ---------------------------------------------------------------- Q8_0 (M:43-56, Q:923-949) */

static float quantize_block32(const float *x, int8_t *qs) {
    float amax = 0.0f;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
    float d = amax / 127.0f;
    float id = d != 0.0f ? 1.0f / d : 0.0f;
    for (int i = 0; i < 32; i++) qs[i] = sat_i8(roundf(x[i] * id));
    return d;
}

void orc_quantize_q8_0(const float *x, void *out, int64_t n) {
    block_q8_0 *y = (block_q8_0 *)out;
    for (int64_t b = 0; b < n / 32; b++) y[b].d = orc_f32_to_f16(quantize_block32(x + 32 * b, y[b].qs));
}

void orc_dequantize_q8_0(const void *in, float *y, int64_t n) { /* Q:905-921 */
    const block_q8_0 *x = (const block_q8_0 *)in;
    for (int64_t b = 0; b < n / 32; b++) {
        float d = orc_f16_to_f32(x[b].d);
        for (int j = 0; j < 32; j++) y[32 * b + j] = (float)x[b].qs[j] * d;
    }
}

/* ---------------------------------------------------------------- Q8_1 activation blocks */

/* The CPU type's quantizer, `BlockQ8_1::from_float` (Q:1031-1060): s = f16(sum of quants) * d in f16. */
void orc_quantize_q8_1_cpu(const float *x, void *out, int64_t n) {
    block_q8_1 *y = (block_q8_1 *)out;
    for (int64_t b = 0; b < n / 32; b++) {
        const float *xs = x + 32 * b;
        float amax = 0.0f;
        for (int j = 0; j < 32; j++) amax = fmaxf(amax, fabsf(xs[j]));
        float d = amax / 127.0f;
        float id = d != 0.0f ? 1.0f / d : 0.0f;
        y[b].d = orc_f32_to_f16(d);
        int sum = 0;
        for (int j = 0; j < 16; j++) {
            y[b].qs[j] = sat_i8(roundf(xs[j] * id));
            y[b].qs[j + 16] = sat_i8(roundf(xs[j + 16] * id));
            sum += y[b].qs[j] + y[b].qs[j + 16];
        }
        /* the half crate multiplies two f16 in f32 and rounds once */
        float s16 = orc_f16_to_f32(orc_f32_to_f16((float)sum));
        y[b].s = orc_f32_to_f16(s16 * orc_f16_to_f32(y[b].d));
    }
}

/* The decode path's activation quantizer, the kernel `mmvq_gguf_quantize_q8_1_*` (CU:9-107): rows of
 * `kx` values padded with zeros to `kx_padded`; per 32: d = amax / 127 (IEEE division), q = roundf(x / d),
 * stored as f16(d) and f16(sum of x) where the sum is the xor-butterfly of a 32-lane warp
 * (offsets 16, 8, 4, 2, 1; mmvq_gguf.cuh:37-43). The reference builds that kernel with fast-math, so
 * its own division is approximate; this oracle and the kernel under test use the exact one. */
void orc_quantize_q8_1_mmvq(const float *x, void *out, int64_t kx, int64_t kx_padded, int64_t rows) {
    block_q8_1 *y = (block_q8_1 *)out;
    int64_t nb = kx_padded / 32;
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t b = 0; b < nb; b++) {
            float v[32], s[32], t[32];
            float amax = 0.0f;
            for (int j = 0; j < 32; j++) {
                int64_t ix = 32 * b + j;
                v[j] = ix < kx ? x[r * kx + ix] : 0.0f;
                amax = fmaxf(amax, fabsf(v[j]));
                s[j] = v[j];
            }
            for (int mask = 16; mask > 0; mask >>= 1) {
                for (int j = 0; j < 32; j++) t[j] = s[j] + s[j ^ mask];
                memcpy(s, t, sizeof s);
            }
            float d = amax / 127.0f;
            block_q8_1 *yb = &y[r * nb + b];
            for (int j = 0; j < 32; j++) yb->qs[j] = amax == 0.0f ? 0 : (int8_t)roundf(v[j] / d);
            yb->d = orc_f32_to_f16(d);
            yb->s = orc_f32_to_f16(s[0]);
        }
    }
}

/* The tensor-core matvec tier's activation layout, `mmvq_tc_quantize`
 * (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_quantize.cu:148-190, layout mmvq_tc_act.cuh:1-7): the rows in
 * halves of 8, one half after the other; per half and with nb = ceil(kx / 32) blocks: nb * 32 int2 fragments (entry
 * 4r + t of a block holds row r's values 4t..4t+3 then 16+4t..16+4t+3), then nb * 8 f16 scales (d = amax / 127), then
 * nb * 8 int16 block sums of the quants. q = roundf(x / d) (IEEE division here, as in orc_quantize_q8_1_mmvq); rows
 * past `rows` and values past `kx` are zero. `out` holds ceil(rows / 8) * nb * 288 bytes. */
void orc_quantize_mmvq_tc(const float *x, void *out, int64_t kx, int64_t rows) {
    int64_t nb = (kx + 31) / 32;
    int64_t halves = (rows + 7) / 8;
    for (int64_t h = 0; h < halves; h++) {
        uint8_t *base = (uint8_t *)out + h * nb * 288;
        int8_t *qs = (int8_t *)base;
        uint16_t *ds = (uint16_t *)(base + nb * 256);
        int16_t *ss = (int16_t *)(base + nb * 256 + nb * 16);
        for (int64_t b = 0; b < nb; b++) {
            for (int r = 0; r < 8; r++) {
                int64_t row = h * 8 + r;
                float v[32];
                float amax = 0.0f;
                for (int j = 0; j < 32; j++) {
                    int64_t col = 32 * b + j;
                    v[j] = (row < rows && col < kx) ? x[row * kx + col] : 0.0f;
                    amax = fmaxf(amax, fabsf(v[j]));
                }
                float d = amax / 127.0f;
                int sum = 0;
                for (int j = 0; j < 32; j++) {
                    int8_t q = amax == 0.0f ? 0 : (int8_t)roundf(v[j] / d);
                    sum += q;
                    int t = (j & 15) >> 2;
                    qs[b * 256 + (4 * r + t) * 8 + (j >= 16 ? 4 : 0) + (j & 3)] = q;
                }
                ds[b * 8 + r] = orc_f32_to_f16(d);
                ss[b * 8 + r] = (int16_t)sum;
            }
        }
    }
}

/* The prefill path's activation quantizer, `quantize_mmq_q8_1` (MQ:98-199): blocks of 128 values of one
 * token, 144 bytes: 16 bytes of scales then 128 int8. Block index ib = (k / 128) * rows + row.
 * layout 0 (D4): four f32 d; layout 1 (DS4): four half2 (d, sum of x). d_inv = 127 / amax,
 * q = roundf(x * d_inv), d = 1 / d_inv (0 when amax is 0). The sum is the 8-lane xor-butterfly of
 * per-thread 4-value sums (each thread holds 4 consecutive values, 8 threads a block of 32). */
void orc_quantize_q8_1_mmq(const float *x, void *out, int64_t kx, int64_t kx_padded, int64_t rows, int layout) {
    uint8_t *y = (uint8_t *)out;
    int64_t nb128 = kx_padded / 128;
    for (int64_t r = 0; r < rows; r++) {
        for (int64_t kb = 0; kb < nb128; kb++) {
            uint8_t *blk = y + (kb * rows + r) * 144;
            for (int sub = 0; sub < 4; sub++) {
                float v[32];
                float amax = 0.0f;
                for (int j = 0; j < 32; j++) {
                    int64_t ix = kb * 128 + sub * 32 + j;
                    v[j] = ix < kx ? x[r * kx + ix] : 0.0f;
                    amax = fmaxf(amax, fabsf(v[j]));
                }
                float ps[8], pt[8];
                for (int t = 0; t < 8; t++) ps[t] = v[4 * t] + v[4 * t + 1] + v[4 * t + 2] + v[4 * t + 3];
                for (int mask = 4; mask > 0; mask >>= 1) {
                    for (int t = 0; t < 8; t++) pt[t] = ps[t] + ps[t ^ mask];
                    memcpy(ps, pt, sizeof ps);
                }
                float d_inv = 127.0f / amax;
                int8_t *qs = (int8_t *)(blk + 16 + 32 * sub);
                for (int j = 0; j < 32; j++) qs[j] = amax == 0.0f ? 0 : (int8_t)roundf(v[j] * d_inv);
                float d = amax == 0.0f ? 0.0f : 1.0f / d_inv;
                if (layout == 0) {
                    memcpy(blk + 4 * sub, &d, 4);
                } else {
                    uint16_t hd = orc_f32_to_f16(d), hs = orc_f32_to_f16(ps[0]);
                    memcpy(blk + 4 * sub, &hd, 2);
                    memcpy(blk + 4 * sub + 2, &hs, 2);
                }
            }
        }
    }
}

/* ---------------------------------------------------------------- Q8_K (Q:2721-2760) */

void orc_quantize_q8_k(const float *x, void *out, int64_t n) {
    block_q8_k *y = (block_q8_k *)out;
    for (int64_t b = 0; b < n / QK_K; b++) {
        const float *xs = x + QK_K * b;
        float max = 0.0f, amax = 0.0f;
        for (int j = 0; j < QK_K; j++) {
            if (amax < fabsf(xs[j])) { amax = fabsf(xs[j]); max = xs[j]; }
        }
        if (amax == 0.0f) {
            y[b].d = 0.0f;
            memset(y[b].qs, 0, sizeof y[b].qs);
            memset(y[b].bsums, 0, sizeof y[b].bsums);
            continue;
        }
        float iscale = -127.0f / max;
        for (int j = 0; j < QK_K; j++) {
            float v = roundf(iscale * xs[j]);
            v = v < -128.0f ? -128.0f : (v > 127.0f ? 127.0f : v);
            y[b].qs[j] = (int8_t)v;
        }
        for (int j = 0; j < QK_K / 16; j++) {
            int sum = 0;
            for (int ii = 0; ii < 16; ii++) sum += y[b].qs[16 * j + ii];
            y[b].bsums[j] = (int16_t)sum;
        }
        y[b].d = 1.0f / iscale;
    }
}

/* ---------------------------------------------------------------- scale searches */

/* `make_qx_quants` (U:135-264). ik = the IkLlama mode (fused multiply-adds and the extra search). */
static float make_qx_quants(int n, int nmax, const float *x, int8_t *ls, int rmse_type, const float *qw, int ik) {
    float max = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; i++) {
        if (fabsf(x[i]) > amax) { amax = fabsf(x[i]); max = x[i]; }
    }
    if (amax < GROUP_MAX_EPS) {
        for (int i = 0; i < n; i++) ls[i] = 0;
        return 0.0f;
    }
#define QX_QUANT(isc, v) clampi(nearest_int_mul(ik, (isc), (v)), -nmax, nmax - 1)
    float iscale = -(float)nmax / max;
    if (rmse_type == 0) {
        for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + QX_QUANT(iscale, x[i]));
        return 1.0f / iscale;
    }
    int return_early = rmse_type < 0;
    rmse_type = abs(rmse_type);
    float w[64];
    for (int i = 0; i < n; i++) {
        if (qw) w[i] = qw[i];
        else if (rmse_type == 1) w[i] = x[i] * x[i];
        else if (rmse_type == 2) w[i] = 1.0f;
        else if (rmse_type == 3) w[i] = fabsf(x[i]);
        else w[i] = sqrtf(fabsf(x[i]));
    }
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; i++) { /* first pass fuses as the mode says */
        float l = (float)QX_QUANT(iscale, x[i]);
        sumlx = madd(ik, w[i] * x[i], l, sumlx);
        suml2 = madd(ik, w[i] * l, l, suml2);
    }
    for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + QX_QUANT(iscale, x[i]));
    float scale = suml2 != 0.0f ? sumlx / suml2 : 0.0f;
    if (return_early) return suml2 > 0.0f ? 0.5f * (scale + 1.0f / iscale) : 1.0f / iscale;
    float best = scale * sumlx;
    float best_sumlx = sumlx, best_suml2 = suml2;
    for (int is = -9; is <= 9; is++) {
        float tenths = (float)is;
        float cand[2];
        int ncand = 0;
        if (is != 0 || ik) cand[ncand++] = -madd(ik, 0.1f, tenths, (float)nmax) / max;
        if (ik) cand[ncand++] = madd(ik, 0.1f, tenths, (float)(nmax - 1)) / max;
        for (int c = 0; c < ncand; c++) {
            float isc = cand[c];
            sumlx = 0.0f; suml2 = 0.0f;
            for (int i = 0; i < n; i++) { /* later passes never fuse */
                float l = (float)QX_QUANT(isc, x[i]);
                sumlx = w[i] * x[i] * l + sumlx;
                suml2 = w[i] * l * l + suml2;
            }
            if (suml2 > 0.0f && sumlx * sumlx > best * suml2) {
                for (int i = 0; i < n; i++) ls[i] = (int8_t)(nmax + QX_QUANT(isc, x[i]));
                scale = sumlx / suml2;
                best = scale * sumlx;
                best_sumlx = sumlx; best_suml2 = suml2;
            }
        }
    }
    if (!ik) return scale;
    sumlx = best_sumlx; suml2 = best_suml2;
    for (int iter = 0; iter < n * (2 * nmax - 1); iter++) {
        float abs_gmax = 0.0f, gmax = 0.0f;
        int best_j = -1;
        for (int j = 0; j < n; j++) {
            int l = ls[j] - nmax;
            float g = scale * w[j] * madd(ik, -scale, (float)l, x[j]);
            int movable = (g > 0.0f && l < nmax - 1) || (g < 0.0f && l > -nmax);
            if (movable && fabsf(g) > abs_gmax) { abs_gmax = fabsf(g); gmax = g; best_j = j; }
        }
        if (best_j < 0) break;
        int j = best_j;
        int l = ls[j] - nmax;
        float new_sumlx, new_suml2;
        if (gmax > 0.0f) {
            l += 1;
            new_sumlx = sumlx + w[j] * x[j];
            new_suml2 = madd(ik, w[j], (float)(2 * l - 1), suml2);
        } else {
            l -= 1;
            new_sumlx = sumlx - w[j] * x[j];
            new_suml2 = madd(ik, -w[j], (float)(2 * l + 1), suml2);
        }
        if (new_suml2 > 0.0f && new_sumlx * new_sumlx > best * new_suml2) {
            sumlx = new_sumlx; suml2 = new_suml2;
            scale = sumlx / suml2;
            best = scale * sumlx;
            ls[j] = (int8_t)(l + nmax);
        } else {
            break;
        }
    }
    return scale;
#undef QX_QUANT
}

/* `make_qkx2_quants` (U:268-361); returns scale, writes the negated min to *the_min. */
static float make_qkx2_quants(int n, int nmax, const float *x, const float *weights, float rmin, float rdelta,
                              int nstep, int use_mad, uint8_t *L, float *the_min, int ik) {
    float min = x[0], max = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; i++) {
        min = fminf(min, x[i]);
        max = fmaxf(max, x[i]);
        sum_w += weights[i];
        sum_x = madd(ik, weights[i], x[i], sum_x);
    }
    if (min > 0.0f) min = 0.0f;
    int flat = ik ? (max - min < QKX_FLAT_RANGE) : (max == min);
    if (flat) {
        for (int i = 0; i < n; i++) L[i] = 0;
        *the_min = -min;
        return 0.0f;
    }
    float iscale = (float)nmax / (max - min);
    float scale = 1.0f / iscale;
    float best_error = 0.0f;
    for (int i = 0; i < n; i++) {
        int li = clampi(nearest_int_mul(ik, iscale, x[i] - min), 0, nmax);
        L[i] = (uint8_t)li;
        float diff = madd(ik, scale, (float)li, min) - x[i];
        diff = use_mad ? fabsf(diff) : diff * diff;
        best_error = madd(ik, weights[i], diff, best_error);
    }
    if (nstep == 0) { *the_min = -min; return scale; }
    int laux[64];
    for (int is = 0; is <= nstep; is++) {
        iscale = (madd(ik, rdelta, (float)is, rmin) + (float)nmax) / (max - min);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; i++) {
            int li = clampi(nearest_int_mul(ik, iscale, x[i] - min), 0, nmax);
            laux[i] = li;
            float wl = weights[i] * (float)li;
            sum_l += wl;
            sum_l2 = madd(ik, wl, (float)li, sum_l2);
            sum_xl = madd(ik, wl, x[i], sum_xl);
        }
        float d = msub(ik, sum_w, sum_l2, sum_l, sum_l);
        if (d > 0.0f) {
            float this_scale = -msub(ik, sum_x, sum_l, sum_w, sum_xl) / d;
            float this_min = msub(ik, sum_l2, sum_x, sum_l, sum_xl) / d;
            if (this_min > 0.0f) {
                this_min = 0.0f;
                this_scale = sum_xl / sum_l2;
            }
            float cur_error = 0.0f;
            for (int i = 0; i < n; i++) {
                float diff = madd(ik, this_scale, (float)laux[i], this_min) - x[i];
                diff = use_mad ? fabsf(diff) : diff * diff;
                cur_error = madd(ik, weights[i], diff, cur_error);
            }
            if (cur_error < best_error) {
                for (int i = 0; i < n; i++) L[i] = (uint8_t)laux[i];
                best_error = cur_error;
                scale = this_scale;
                min = this_min;
            }
        }
    }
    *the_min = -min;
    return scale;
}

static inline void get_scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m) { /* U:119-129 */
    if (j < 4) {
        *d = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *d = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ---------------------------------------------------------------- Q4_K (Q:1930-2015, no importance matrix) */

static void quantize_q4_k_block(const float *x, block_q4_k *block, int ik) {
    uint8_t L[QK_K];
    float mins[8], scales[8];
    memset(block, 0, sizeof *block);
    for (int j = 0; j < 8; j++) {
        const float *xs = x + 32 * j;
        float sumsq = 0.0f;
        for (int i = 0; i < 32; i++) sumsq = sumsq + xs[i] * xs[i]; /* Q:302-305 */
        float av_x = sqrtf(sumsq / 32.0f);
        float weights[32];
        for (int i = 0; i < 32; i++) weights[i] = av_x + fabsf(xs[i]);
        scales[j] = make_qkx2_quants(32, 15, xs, weights, -1.0f, 0.1f, 20, 0, L + 32 * j, &mins[j], ik);
    }
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; j++) {
        max_scale = fmaxf(scales[j], max_scale);
        max_min = fmaxf(mins[j], max_min);
    }
    float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
    float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
    for (int j = 0; j < 8; j++) {
        int lsi = nearest_int_mul(ik, inv_scale, scales[j]);
        int lmi = nearest_int_mul(ik, inv_min, mins[j]);
        uint8_t ls = (uint8_t)(lsi < 63 ? lsi : 63);
        uint8_t lm = (uint8_t)(lmi < 63 ? lmi : 63);
        if (j < 4) {
            block->scales[j] = ls;
            block->scales[j + 4] = lm;
        } else {
            block->scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
            block->scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
            block->scales[j] |= (uint8_t)((lm >> 4) << 6);
        }
    }
    block->d = orc_f32_to_f16(max_scale / 63.0f);
    block->dmin = orc_f32_to_f16(max_min / 63.0f);
    for (int j = 0; j < 8; j++) {
        uint8_t sc, m;
        get_scale_min_k4(j, block->scales, &sc, &m);
        float d = orc_f16_to_f32(block->d) * (float)sc;
        if (d != 0.0f) {
            float dm = orc_f16_to_f32(block->dmin) * (float)m;
            for (int ii = 0; ii < 32; ii++) {
                int l = nearest_int((x[32 * j + ii] + dm) / d);
                L[32 * j + ii] = (uint8_t)clampi(l, 0, 15);
            }
        }
    }
    for (int j = 0; j < QK_K; j += 64)
        for (int l = 0; l < 32; l++) block->qs[(j / 64) * 32 + l] = (uint8_t)(L[j + l] | (L[j + l + 32] << 4));
}

void orc_quantize_q4_k(const float *x, void *out, int64_t n, int mode) {
    block_q4_k *y = (block_q4_k *)out;
    int64_t nb = n / QK_K;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) quantize_q4_k_block(x + QK_K * b, &y[b], mode == ORC_IKLLAMA);
}

void orc_dequantize_q4_k(const void *in, float *y, int64_t n) { /* Q:2096-2123 */
    const block_q4_k *x = (const block_q4_k *)in;
    for (int64_t b = 0; b < n / QK_K; b++) {
        float d = orc_f16_to_f32(x[b].d), min = orc_f16_to_f32(x[b].dmin);
        float *yb = y + QK_K * b;
        int is = 0, yi = 0;
        for (int j = 0; j < QK_K; j += 64) {
            const uint8_t *q = x[b].qs + j / 2;
            uint8_t sc, m;
            get_scale_min_k4(is, x[b].scales, &sc, &m);
            float d1 = d * (float)sc, m1 = min * (float)m;
            get_scale_min_k4(is + 1, x[b].scales, &sc, &m);
            float d2 = d * (float)sc, m2 = min * (float)m;
            for (int l = 0; l < 32; l++) yb[yi++] = d1 * (float)(q[l] & 0xF) - m1;
            for (int l = 0; l < 32; l++) yb[yi++] = d2 * (float)(q[l] >> 4) - m2;
            is += 2;
        }
    }
}

/* ---------------------------------------------------------------- Q6_K (Q:2577-2680) */

/* imatrix: NULL, or `n_per_row` importance weights; superblock b of a row uses imatrix[256 * (b % (n_per_row/256))..]. */
void orc_quantize_q6_k(const float *x, void *out, int64_t n, const float *imatrix, int64_t n_per_row, int mode) {
    block_q6_k *y = (block_q6_k *)out;
    int ik = mode == ORC_IKLLAMA;
    int64_t nb = n / QK_K;
#pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < nb; b++) {
        /* the reference keeps `l` across superblocks; every entry is rewritten by make_qx_quants each time,
         * so a per-block array is the same thing */
        int8_t L[QK_K];
        float scales[16];
        const float *xb = x + QK_K * b;
        const float *qw = imatrix ? imatrix + QK_K * (b % (n_per_row / QK_K)) : NULL;
        float max_scale = 0.0f, max_abs_scale = 0.0f;
        for (int ib = 0; ib < 16; ib++) {
            float scale = make_qx_quants(16, 32, xb + 16 * ib, L + 16 * ib, 1, qw ? qw + 16 * ib : NULL, ik);
            scales[ib] = scale;
            if (fabsf(scale) > max_abs_scale) { max_abs_scale = fabsf(scale); max_scale = scale; }
        }
        float iscale = -128.0f / max_scale;
        y[b].d = orc_f32_to_f16(1.0f / iscale);
        for (int ib = 0; ib < 16; ib++) {
            int v = nearest_int_mul(ik, iscale, scales[ib]);
            y[b].scales[ib] = (int8_t)(v < 127 ? v : 127);
        }
        for (int j = 0; j < 16; j++) {
            float d = orc_f16_to_f32(y[b].d) * (float)y[b].scales[j];
            if (d == 0.0f) continue;
            for (int ii = 0; ii < 16; ii++)
                L[16 * j + ii] = (int8_t)(clampi(nearest_int(xb[16 * j + ii] / d), -32, 31) + 32);
        }
        for (int h = 0; h < 2; h++) {
            uint8_t *ql = y[b].ql + 64 * h, *qh = y[b].qh + 32 * h;
            const int8_t *l = L + 128 * h;
            for (int i = 0; i < 32; i++) {
                int q1 = l[i], q2 = l[i + 32], q3 = l[i + 64], q4 = l[i + 96];
                ql[i] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4));
                ql[i + 32] = (uint8_t)((q2 & 0xF) | ((q4 & 0xF) << 4));
                qh[i] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
            }
        }
    }
}

void orc_dequantize_q6_k(const void *in, float *y, int64_t n) { /* Q:2649-2680 */
    const block_q6_k *x = (const block_q6_k *)in;
    for (int64_t b = 0; b < n / QK_K; b++) {
        float d = orc_f16_to_f32(x[b].d);
        for (int h = 0; h < 2; h++) {
            float *ys = y + QK_K * b + 128 * h;
            const int8_t *sc = x[b].scales + 8 * h;
            const uint8_t *ql = x[b].ql + 64 * h, *qh = x[b].qh + 32 * h;
            for (int l = 0; l < 32; l++) {
                int is = l / 16;
                int8_t q1 = (int8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
                int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
                int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
                int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
                ys[l] = d * (float)sc[is] * (float)q1;
                ys[l + 32] = d * (float)sc[is + 2] * (float)q2;
                ys[l + 64] = d * (float)sc[is + 4] * (float)q3;
                ys[l + 96] = d * (float)sc[is + 6] * (float)q4;
            }
        }
    }
}

/* ---------------------------------------------------------------- vec_dot_unopt */

static float vec_dot_q8_0_q8_0(int64_t n, const block_q8_0 *xs, const block_q8_0 *ys) { /* Q:981-999 */
    float sumf = 0.0f;
    for (int64_t b = 0; b < n / 32; b++) {
        int sum_i = 0;
        for (int j = 0; j < 32; j++) sum_i += (int)xs[b].qs[j] * (int)ys[b].qs[j];
        sumf += (float)sum_i * orc_f16_to_f32(xs[b].d) * orc_f16_to_f32(ys[b].d);
    }
    return sumf;
}

static float vec_dot_q4_k_q8_k(int64_t n, const block_q4_k *xs, const block_q8_k *ys) { /* Q:1848-1928 */
    int8_t aux8[QK_K];
    int16_t aux16[8];
    float sums[8] = {0};
    int32_t aux32[8];
    float sumf = 0.0f;
    for (int64_t b = 0; b < n / QK_K; b++) {
        const block_q4_k *x = &xs[b];
        const block_q8_k *y = &ys[b];
        memset(aux32, 0, sizeof aux32);
        int8_t *a = aux8;
        const uint8_t *q4 = x->qs;
        for (int j = 0; j < QK_K / 64; j++) {
            for (int l = 0; l < 32; l++) a[l] = (int8_t)(q4[l] & 0xF);
            a += 32;
            for (int l = 0; l < 32; l++) a[l] = (int8_t)(q4[l] >> 4);
            a += 32;
            q4 += 32;
        }
        uint8_t scales[8], mins[8];
        for (int j = 0; j < 8; j++) get_scale_min_k4(j, x->scales, &scales[j], &mins[j]);
        int sumi = 0;
        for (int j = 0; j < QK_K / 16; j++) sumi += (int)y->bsums[j] * (int)mins[j / 2];
        a = aux8;
        const int8_t *q8 = y->qs;
        for (int is = 0; is < 8; is++) {
            int32_t scale = scales[is];
            for (int r = 0; r < 4; r++) {
                for (int l = 0; l < 8; l++) aux16[l] = (int16_t)((int16_t)q8[l] * (int16_t)a[l]);
                for (int l = 0; l < 8; l++) aux32[l] += scale * (int32_t)aux16[l];
                q8 += 8;
                a += 8;
            }
        }
        float d = orc_f16_to_f32(x->d) * y->d;
        for (int l = 0; l < 8; l++) sums[l] += d * (float)aux32[l];
        float dmin = orc_f16_to_f32(x->dmin) * y->d;
        sumf -= dmin * (float)sumi;
    }
    float tail = 0.0f;
    for (int l = 0; l < 8; l++) tail += sums[l];
    return sumf + tail;
}

static float vec_dot_q6_k_q8_k(int64_t n, const block_q6_k *xs, const block_q8_k *ys) { /* Q:2518-2575 */
    int8_t aux8[QK_K];
    int16_t aux16[8];
    float sums[8] = {0};
    float aux32[8];
    for (int64_t b = 0; b < n / QK_K; b++) {
        const block_q6_k *x = &xs[b];
        const block_q8_k *y = &ys[b];
        memset(aux32, 0, sizeof aux32);
        for (int j = 0; j < QK_K; j += 128) {
            int8_t *a = aux8 + j;
            const uint8_t *q4 = x->ql + j / 2, *qh = x->qh + j / 4;
            for (int l = 0; l < 32; l++) {
                a[l] = (int8_t)((int)((q4[l] & 0xF) | ((qh[l] & 3) << 4)) - 32);
                a[l + 32] = (int8_t)((int)((q4[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32);
                a[l + 64] = (int8_t)((int)((q4[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32);
                a[l + 96] = (int8_t)((int)((q4[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32);
            }
        }
        for (int j = 0; j < 16; j++) {
            float scale = (float)x->scales[j];
            const int8_t *q8 = y->qs + 16 * j;
            const int8_t *a = aux8 + 16 * j;
            for (int l = 0; l < 8; l++) aux16[l] = (int16_t)((int16_t)q8[l] * (int16_t)a[l]);
            for (int l = 0; l < 8; l++) aux32[l] += scale * (float)aux16[l];
            q8 += 8;
            a += 8;
            for (int l = 0; l < 8; l++) aux16[l] = (int16_t)((int16_t)q8[l] * (int16_t)a[l]);
            for (int l = 0; l < 8; l++) aux32[l] += scale * (float)aux16[l];
        }
        float d = orc_f16_to_f32(x->d) * y->d;
        for (int l = 0; l < 8; l++) sums[l] += aux32[l] * d;
    }
    float total = 0.0f;
    for (int l = 0; l < 8; l++) total += sums[l];
    return total;
}

/* ---------------------------------------------------------------- matmul (Q:2777-2894) */

static int64_t type_block_elems(int t) { return t == ORC_Q8_0 ? 32 : QK_K; }
static int64_t type_block_bytes(int t) { return t == ORC_Q8_0 ? 34 : (t == ORC_Q4_K ? 144 : (t == ORC_Q6_K ? 210 : 0)); }

int64_t orc_type_block_elems(int t) { return type_block_elems(t); }
int64_t orc_type_block_bytes(int t) { return type_block_bytes(t); }

/* dst[m][n] = lhs[m][k] . rhs[n][k]^T with each lhs row quantized to the weight type's dot type
 * (Q8_K for Q4_K / Q6_K, Q8_0 for Q8_0) and one integer vec_dot per output. Returns 0, or -1 for a bad type. */
int orc_matmul(int type, int64_t m, int64_t k, int64_t n, const float *lhs, const void *rhs, float *dst, int threads) {
    int64_t bs = type_block_elems(type), bb = type_block_bytes(type);
    if (bb == 0 || k % bs != 0) return -1;
    int64_t kb = k / bs;
    int64_t act_bytes = type == ORC_Q8_0 ? 34 : 292;
    uint8_t *lhs_q = (uint8_t *)malloc((size_t)(m * kb * act_bytes));
    if (!lhs_q) return -2;
    for (int64_t r = 0; r < m; r++) {
        if (type == ORC_Q8_0) orc_quantize_q8_0(lhs + r * k, lhs_q + r * kb * act_bytes, k);
        else orc_quantize_q8_k(lhs + r * k, lhs_q + r * kb * act_bytes, k);
    }
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#else
    int nt = 1;
    (void)threads;
#endif
    for (int64_t r = 0; r < m; r++) {
        const uint8_t *lrow = lhs_q + r * kb * act_bytes;
#pragma omp parallel for schedule(static) num_threads(nt)
        for (int64_t c = 0; c < n; c++) {
            const uint8_t *wrow = (const uint8_t *)rhs + c * kb * bb;
            float v;
            if (type == ORC_Q8_0) v = vec_dot_q8_0_q8_0(k, (const block_q8_0 *)wrow, (const block_q8_0 *)lrow);
            else if (type == ORC_Q4_K) v = vec_dot_q4_k_q8_k(k, (const block_q4_k *)wrow, (const block_q8_k *)lrow);
            else v = vec_dot_q6_k_q8_k(k, (const block_q6_k *)wrow, (const block_q8_k *)lrow);
            dst[r * n + c] = v;
        }
    }
    free(lhs_q);
    return 0;
}

/* The decode kernels' own arithmetic, accumulated in double: weights times Q8_1 activation blocks
 * (`acts`: [m][k_padded/32] blocks of 36 bytes as orc_quantize_q8_1_mmvq writes them). Per 32 values:
 *   Q4_K: d*sc*d8*sum(q*q8) - dmin*m*d8*sum(q8);  Q6_K: d*sc16*d8*sum((q-32)*q8) per 16;  Q8_0: d*d8*sum(q*q8).
 * A GEMV fed the same blocks differs from this only by f32 rounding and summation order. */
int orc_matmul_q8_1(int type, int64_t m, int64_t k, int64_t k_padded, int64_t n, const void *acts, const void *rhs,
                    double *dst, int threads) {
    int64_t bs = type_block_elems(type), bb = type_block_bytes(type);
    if (bb == 0 || k % bs != 0) return -1;
    int64_t kb = k / bs, anb = k_padded / 32;
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#else
    int nt = 1;
    (void)threads;
#endif
#pragma omp parallel for schedule(static) num_threads(nt)
    for (int64_t c = 0; c < n; c++) {
        const uint8_t *wrow = (const uint8_t *)rhs + c * kb * bb;
        for (int64_t r = 0; r < m; r++) {
            const block_q8_1 *a = (const block_q8_1 *)acts + r * anb;
            double acc = 0.0;
            if (type == ORC_Q8_0) {
                const block_q8_0 *w = (const block_q8_0 *)wrow;
                for (int64_t b = 0; b < kb; b++) {
                    int s = 0;
                    for (int j = 0; j < 32; j++) s += (int)w[b].qs[j] * (int)a[b].qs[j];
                    acc += (double)orc_f16_to_f32(w[b].d) * (double)orc_f16_to_f32(a[b].d) * (double)s;
                }
            } else if (type == ORC_Q4_K) {
                const block_q4_k *w = (const block_q4_k *)wrow;
                for (int64_t b = 0; b < kb; b++) {
                    double d = orc_f16_to_f32(w[b].d), dmin = orc_f16_to_f32(w[b].dmin);
                    for (int j = 0; j < 8; j++) {
                        uint8_t sc, mn;
                        get_scale_min_k4(j, w[b].scales, &sc, &mn);
                        const block_q8_1 *ab = &a[8 * b + j];
                        const uint8_t *q = w[b].qs + 32 * (j / 2);
                        int dot = 0, s8 = 0;
                        for (int l = 0; l < 32; l++) {
                            int qv = (j & 1) ? (q[l] >> 4) : (q[l] & 0xF);
                            dot += qv * (int)ab->qs[l];
                            s8 += ab->qs[l];
                        }
                        double d8 = orc_f16_to_f32(ab->d);
                        acc += d * sc * d8 * dot - dmin * mn * d8 * s8;
                    }
                }
            } else {
                const block_q6_k *w = (const block_q6_k *)wrow;
                for (int64_t b = 0; b < kb; b++) {
                    double d = orc_f16_to_f32(w[b].d);
                    for (int e = 0; e < QK_K; e++) {
                        int h = e / 128, r128 = e % 128, quad = r128 / 32, l = r128 % 32;
                        const uint8_t *ql = w[b].ql + 64 * h, *qh = w[b].qh + 32 * h;
                        int lo = (quad & 1) ? ql[l + 32] : ql[l];
                        lo = (quad & 2) ? (lo >> 4) : (lo & 0xF);
                        int hi = (qh[l] >> (2 * quad)) & 3;
                        int qv = (lo | (hi << 4)) - 32;
                        const block_q8_1 *ab = &a[8 * b + e / 32];
                        acc += d * (double)w[b].scales[e / 16] * (double)orc_f16_to_f32(ab->d) *
                               (double)(qv * (int)ab->qs[e % 32]);
                    }
                }
            }
            dst[r * n + c] = acc;
        }
    }
    return 0;
}

/* x . dequant(W)^T in double: the "dense" comparator the reference's own tolerance tests use (M:1883-1918). */
int orc_matmul_dense(int type, int64_t m, int64_t k, int64_t n, const float *lhs, const void *rhs, double *dst,
                     int threads) {
    int64_t bs = type_block_elems(type), bb = type_block_bytes(type);
    if (bb == 0 || k % bs != 0) return -1;
    int64_t kb = k / bs;
#ifdef _OPENMP
    int nt = threads > 0 ? threads : omp_get_max_threads();
#else
    int nt = 1;
    (void)threads;
#endif
#pragma omp parallel num_threads(nt)
    {
        float *row = (float *)malloc((size_t)k * sizeof(float));
#pragma omp for schedule(static)
        for (int64_t c = 0; c < n; c++) {
            const uint8_t *wrow = (const uint8_t *)rhs + c * kb * bb;
            if (type == ORC_Q8_0) orc_dequantize_q8_0(wrow, row, k);
            else if (type == ORC_Q4_K) orc_dequantize_q4_k(wrow, row, k);
            else orc_dequantize_q6_k(wrow, row, k);
            for (int64_t r = 0; r < m; r++) {
                double acc = 0.0;
                for (int64_t i = 0; i < k; i++) acc += (double)lhs[r * k + i] * (double)row[i];
                dst[r * n + c] = acc;
            }
        }
        free(row);
    }
    return 0;
}

/* Quantize `rows` rows of `k` f32 values to `type` (default llama.cpp mode unless mode says otherwise). */
int orc_quantize(int type, const float *x, void *out, int64_t rows, int64_t k, int mode) {
    int64_t n = rows * k;
    if (type == ORC_Q8_0) {
        if (k % 32) return -1;
#pragma omp parallel for schedule(static)
        for (int64_t r = 0; r < rows; r++) orc_quantize_q8_0(x + r * k, (uint8_t *)out + r * (k / 32) * 34, k);
        return 0;
    }
    if (k % QK_K) return -1;
    if (type == ORC_Q4_K) { orc_quantize_q4_k(x, out, n, mode); return 0; }
    if (type == ORC_Q6_K) { orc_quantize_q6_k(x, out, n, NULL, k, mode); return 0; }
    return -1;
}

int orc_dequantize(int type, const void *in, float *y, int64_t n) {
    if (type == ORC_Q8_0) orc_dequantize_q8_0(in, y, n);
    else if (type == ORC_Q4_K) orc_dequantize_q4_k(in, y, n);
    else if (type == ORC_Q6_K) orc_dequantize_q6_k(in, y, n);
    else return -1;
    return 0;
}

uint64_t orc_fnv1a64(const uint8_t *bytes, int64_t n) { /* requantize.rs:1095-1099 */
    uint64_t h = 0xcbf29ce484222325ull;
    for (int64_t i = 0; i < n; i++) h = (h ^ bytes[i]) * 0x00000100000001b3ull;
    return h;
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

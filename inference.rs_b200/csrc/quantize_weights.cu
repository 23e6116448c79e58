// Weight quantizers and dequantizers on the device: f32 rows -> packed Q8_0 / Q4_K / Q6_K blocks, byte for byte what the
// reference's CPU quantizer produces in its default mode (`Quantizer::LlamaCpp`, no importance matrix), and back.
//
// Reference: `QTensor::quantize` (crates/inference-tensor/src/quantized/mod.rs:903-918) -> `BlockQ8_0::from_float`
// (k_quants.rs:923-949 via quantize_block32, mod.rs:43-56), `BlockQ4K::quantize_with` (k_quants.rs:1949-2015) with
// `make_qkx2_quants` (utils.rs:268-361), `BlockQ6K::quantize_with` (k_quants.rs:2590-2646) with `make_qx_quants`
// (utils.rs:135-264); `to_float` (k_quants.rs:905-921,2096-2123,2649-2680); the embedding row gather `get_rows`
// (crates/inference-tensor/src/quantized/cuda.rs:151-242). The reference runs the K-quant searches on the host even
// for CUDA tensors (cuda.rs:340-361) and has device quantizers for Q6_K / Q8_0 only
// (crates/inference-quant/kernels/cuda/gguf_quantize/k_quantize_instance_ggufq.cu:1-6).
//
// The scale searches compare sums of f32 products whose rounding decides which candidate wins, so the arithmetic is
// the reference's operation for operation: this file is compiled with -fmad=false (no multiply-add contraction, as the
// reference's LlamaCpp mode, utils.rs:37-45), divisions and square roots are IEEE, and sums run in the same order.
// One thread packs one block (32 values for Q8_0, a 256-value superblock otherwise): the searches are sequential per
// sub-block, and a matrix has hundreds of thousands of blocks.
#include "common.cuh"
#include "runtime.h"

namespace b200q {

constexpr float ROUNDING_MAGIC = 12582912.0f;  // 1.5 * 2^23: adding it rounds to the nearest integer, ties to even
constexpr float GROUP_MAX_EPS = 1e-15f;

__device__ __forceinline__ int nearest_int(float v) {  // utils.rs:32-35
    const float r = v + ROUNDING_MAGIC;
    return (int)(__float_as_uint(r) & 0x007fffffu) - 0x00400000;
}
__device__ __forceinline__ int nearest_int_mul(float a, float b) { return nearest_int(a * b); }  // utils.rs:70-73, unfused
__device__ __forceinline__ int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
__device__ __forceinline__ unsigned short f16_bits(float v) { return __half_as_ushort(__float2half_rn(v)); }
__device__ __forceinline__ float f16_value(unsigned short b) { return __half2float(__ushort_as_half(b)); }
// Rust's `as i8` on a float: saturating, NaN -> 0
__device__ __forceinline__ int sat_i8(float v) {
    if (v != v) return 0;
    if (v <= -128.0f) return -128;
    if (v >= 127.0f) return 127;
    return (int)v;
}

// ---------------------------------------------------------------------------------------------
// Q8_0: d = amax / 127, q = round_half_away(x * (1 / d))
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_q8_0_kernel(const float* __restrict__ x, uint8_t* __restrict__ out, long long nblocks) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float* xb = x + b * 32;
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(xb[i]));
    const float d = amax / 127.0f;
    const float id = d != 0.0f ? 1.0f / d : 0.0f;
    // a block is 34 bytes at a 2-byte-aligned address: seventeen 16-bit stores
    unsigned short* o = reinterpret_cast<unsigned short*>(out + b * Q8_0_BYTES);
    o[0] = f16_bits(d);
    for (int i = 0; i < 16; ++i) {
        const unsigned lo = (unsigned)sat_i8(roundf(xb[2 * i] * id)) & 0xffu;
        const unsigned hi = (unsigned)sat_i8(roundf(xb[2 * i + 1] * id)) & 0xffu;
        o[1 + i] = (unsigned short)(lo | (hi << 8));
    }
}

// ---------------------------------------------------------------------------------------------
// Q4_K
// ---------------------------------------------------------------------------------------------
// make_qkx2_quants(n = 32, nmax = 15, rmin = -1, rdelta = 0.1, nstep = 20, squared error): the weighted least-squares
// search for (scale, min) of one sub-block. Returns the scale; *the_min = -min.
__device__ float search_scale_min_q4(const float* x, const float* weights, uint8_t* L, float* the_min) {
    constexpr int n = 32, nmax = 15, nstep = 20;
    const float rmin = -1.0f, rdelta = 0.1f;
    float mn = x[0], mx = x[0];
    float sum_w = weights[0];
    float sum_x = sum_w * x[0];
    for (int i = 1; i < n; ++i) {
        mn = fminf(mn, x[i]);
        mx = fmaxf(mx, x[i]);
        sum_w += weights[i];
        sum_x = weights[i] * x[i] + sum_x;
    }
    if (mn > 0.0f) mn = 0.0f;
    if (mx == mn) {
        for (int i = 0; i < n; ++i) L[i] = 0;
        *the_min = -mn;
        return 0.0f;
    }
    float iscale = (float)nmax / (mx - mn);
    float scale = 1.0f / iscale;
    float best_error = 0.0f;
    for (int i = 0; i < n; ++i) {
        const int li = clampi(nearest_int_mul(iscale, x[i] - mn), 0, nmax);
        L[i] = (uint8_t)li;
        float diff = (scale * (float)li + mn) - x[i];
        diff = diff * diff;
        best_error = weights[i] * diff + best_error;
    }
    uint8_t laux[n];
    for (int is = 0; is <= nstep; ++is) {
        iscale = ((rdelta * (float)is + rmin) + (float)nmax) / (mx - mn);
        float sum_l = 0.0f, sum_l2 = 0.0f, sum_xl = 0.0f;
        for (int i = 0; i < n; ++i) {
            const int li = clampi(nearest_int_mul(iscale, x[i] - mn), 0, nmax);
            laux[i] = (uint8_t)li;
            const float wl = weights[i] * (float)li;
            sum_l += wl;
            sum_l2 = wl * (float)li + sum_l2;
            sum_xl = wl * x[i] + sum_xl;
        }
        const float d = sum_w * sum_l2 - sum_l * sum_l;
        if (d > 0.0f) {
            float this_scale = -(sum_x * sum_l - sum_w * sum_xl) / d;
            float this_min = (sum_l2 * sum_x - sum_l * sum_xl) / d;
            if (this_min > 0.0f) {
                this_min = 0.0f;
                this_scale = sum_xl / sum_l2;
            }
            float cur_error = 0.0f;
            for (int i = 0; i < n; ++i) {
                float diff = (this_scale * (float)laux[i] + this_min) - x[i];
                diff = diff * diff;
                cur_error = weights[i] * diff + cur_error;
            }
            if (cur_error < best_error) {
                for (int i = 0; i < n; ++i) L[i] = laux[i];
                best_error = cur_error;
                scale = this_scale;
                mn = this_min;
            }
        }
    }
    *the_min = -mn;
    return scale;
}

__device__ __forceinline__ void scale_min_k4(int j, const uint8_t* q, int& sc, int& m) {  // utils.rs:119-129
    if (j < 4) {
        sc = q[j] & 63;
        m = q[j + 4] & 63;
    } else {
        sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
        m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
    }
}

__global__ void __launch_bounds__(64) quantize_q4_k_kernel(const float* __restrict__ xs, uint8_t* __restrict__ out, long long nblocks) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float* x = xs + b * QK_K;
    uint8_t L[QK_K];
    float mins[8], scales[8];
    uint8_t packed_scales[12];
    for (int i = 0; i < 12; ++i) packed_scales[i] = 0;
    for (int j = 0; j < 8; ++j) {
        float xv[32], weights[32];
        float sumsq = 0.0f;
        for (int i = 0; i < 32; ++i) {
            xv[i] = x[32 * j + i];
            sumsq = sumsq + xv[i] * xv[i];  // k_quants.rs:302-305
        }
        const float av_x = sqrtf(sumsq / 32.0f);
        for (int i = 0; i < 32; ++i) weights[i] = av_x + fabsf(xv[i]);
        scales[j] = search_scale_min_q4(xv, weights, L + 32 * j, &mins[j]);
    }
    float max_scale = 0.0f, max_min = 0.0f;
    for (int j = 0; j < 8; ++j) {
        max_scale = fmaxf(scales[j], max_scale);
        max_min = fmaxf(mins[j], max_min);
    }
    const float inv_scale = max_scale > 0.0f ? 63.0f / max_scale : 0.0f;
    const float inv_min = max_min > 0.0f ? 63.0f / max_min : 0.0f;
    for (int j = 0; j < 8; ++j) {
        const int lsi = nearest_int_mul(inv_scale, scales[j]);
        const int lmi = nearest_int_mul(inv_min, mins[j]);
        const uint8_t ls = (uint8_t)(lsi < 63 ? lsi : 63);
        const uint8_t lm = (uint8_t)(lmi < 63 ? lmi : 63);
        if (j < 4) {
            packed_scales[j] = ls;
            packed_scales[j + 4] = lm;
        } else {
            packed_scales[j + 4] = (uint8_t)((ls & 0xF) | ((lm & 0xF) << 4));
            packed_scales[j - 4] |= (uint8_t)((ls >> 4) << 6);
            packed_scales[j] |= (uint8_t)((lm >> 4) << 6);
        }
    }
    const unsigned short dh = f16_bits(max_scale / 63.0f), mh = f16_bits(max_min / 63.0f);
    const float dv = f16_value(dh), mv = f16_value(mh);
    // every value again, against the scales as they are stored (k_quants.rs:1995-2005)
    for (int j = 0; j < 8; ++j) {
        int sc, m;
        scale_min_k4(j, packed_scales, sc, m);
        const float d = dv * (float)sc;
        if (d != 0.0f) {
            const float dm = mv * (float)m;
            for (int ii = 0; ii < 32; ++ii) L[32 * j + ii] = (uint8_t)clampi(nearest_int((x[32 * j + ii] + dm) / d), 0, 15);
        }
    }
    uint8_t* o = out + b * Q4_K_BYTES;
    o[0] = (uint8_t)dh; o[1] = (uint8_t)(dh >> 8);
    o[2] = (uint8_t)mh; o[3] = (uint8_t)(mh >> 8);
    for (int i = 0; i < 12; ++i) o[4 + i] = packed_scales[i];
    for (int c = 0; c < 4; ++c)
        for (int l = 0; l < 32; ++l) o[16 + 32 * c + l] = (uint8_t)(L[64 * c + l] | (L[64 * c + 32 + l] << 4));
}

// ---------------------------------------------------------------------------------------------
// Q6_K
// ---------------------------------------------------------------------------------------------
// make_qx_quants(n = 16, nmax = 32, rmse_type = 1, no importance weights): weights x^2, 18 nudged candidates.
__device__ float search_scale_q6(const float* x, int8_t* ls) {
    constexpr int n = 16, nmax = 32;
    float mx = 0.0f, amax = 0.0f;
    for (int i = 0; i < n; ++i) {
        if (fabsf(x[i]) > amax) {
            amax = fabsf(x[i]);
            mx = x[i];
        }
    }
    if (amax < GROUP_MAX_EPS) {
        for (int i = 0; i < n; ++i) ls[i] = 0;
        return 0.0f;
    }
    float iscale = -(float)nmax / mx;
    float w[n];
    for (int i = 0; i < n; ++i) w[i] = x[i] * x[i];
    float sumlx = 0.0f, suml2 = 0.0f;
    for (int i = 0; i < n; ++i) {
        const float l = (float)clampi(nearest_int_mul(iscale, x[i]), -nmax, nmax - 1);
        sumlx = (w[i] * x[i]) * l + sumlx;
        suml2 = (w[i] * l) * l + suml2;
    }
    for (int i = 0; i < n; ++i) ls[i] = (int8_t)(nmax + clampi(nearest_int_mul(iscale, x[i]), -nmax, nmax - 1));
    float scale = suml2 != 0.0f ? sumlx / suml2 : 0.0f;
    float best = scale * sumlx;
    for (int is = -9; is <= 9; ++is) {
        if (is == 0) continue;
        const float isc = -(0.1f * (float)is + (float)nmax) / mx;
        sumlx = 0.0f;
        suml2 = 0.0f;
        for (int i = 0; i < n; ++i) {
            const float l = (float)clampi(nearest_int_mul(isc, x[i]), -nmax, nmax - 1);
            sumlx = w[i] * x[i] * l + sumlx;
            suml2 = w[i] * l * l + suml2;
        }
        if (suml2 > 0.0f && sumlx * sumlx > best * suml2) {
            for (int i = 0; i < n; ++i) ls[i] = (int8_t)(nmax + clampi(nearest_int_mul(isc, x[i]), -nmax, nmax - 1));
            scale = sumlx / suml2;
            best = scale * sumlx;
        }
    }
    return scale;
}

__global__ void __launch_bounds__(64) quantize_q6_k_kernel(const float* __restrict__ xs, uint8_t* __restrict__ out, long long nblocks) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float* xb = xs + b * QK_K;
    int8_t L[QK_K];
    float scales[16];
    float max_scale = 0.0f, max_abs_scale = 0.0f;
    for (int ib = 0; ib < 16; ++ib) {
        float xv[16];
        for (int i = 0; i < 16; ++i) xv[i] = xb[16 * ib + i];
        const float scale = search_scale_q6(xv, L + 16 * ib);
        scales[ib] = scale;
        if (fabsf(scale) > max_abs_scale) {
            max_abs_scale = fabsf(scale);
            max_scale = scale;
        }
    }
    // an all-zero superblock gives max_scale = 0, iscale = -inf, d = f16(-0.0), scales 0: as the reference
    const float iscale = -128.0f / max_scale;
    const unsigned short dh = f16_bits(1.0f / iscale);
    const float dv = f16_value(dh);
    int8_t sc8[16];
    for (int ib = 0; ib < 16; ++ib) {
        // (-inf * 0 is a NaN whose mantissa bits differ between machines: the reference's host turns it into scale 0)
        const int v = max_abs_scale == 0.0f ? 0 : nearest_int_mul(iscale, scales[ib]);
        sc8[ib] = (int8_t)(v < 127 ? v : 127);
    }
    for (int j = 0; j < 16; ++j) {
        const float d = dv * (float)sc8[j];
        if (d == 0.0f) continue;
        for (int ii = 0; ii < 16; ++ii) L[16 * j + ii] = (int8_t)(clampi(nearest_int(xb[16 * j + ii] / d), -32, 31) + 32);
    }
    uint8_t* o = out + b * Q6_K_BYTES;
    for (int h = 0; h < 2; ++h) {
        uint8_t* ql = o + 64 * h;
        uint8_t* qh = o + 128 + 32 * h;
        const int8_t* l = L + 128 * h;
        for (int i = 0; i < 32; ++i) {
            const int q1 = l[i], q2 = l[i + 32], q3 = l[i + 64], q4 = l[i + 96];
            ql[i] = (uint8_t)((q1 & 0xF) | ((q3 & 0xF) << 4));
            ql[i + 32] = (uint8_t)((q2 & 0xF) | ((q4 & 0xF) << 4));
            qh[i] = (uint8_t)((q1 >> 4) | ((q2 >> 4) << 2) | ((q3 >> 4) << 4) | ((q4 >> 4) << 6));
        }
    }
    for (int ib = 0; ib < 16; ++ib) o[192 + ib] = (uint8_t)sc8[ib];
    o[208] = (uint8_t)dh;
    o[209] = (uint8_t)(dh >> 8);
}

// ---------------------------------------------------------------------------------------------
// to_float and the row gather: one thread per 32 values
// ---------------------------------------------------------------------------------------------
template <typename T>
__device__ void dequant_group32(int type, const uint8_t* row, int g, T* dst) {
    if (type == TYPE_Q8_0) {
        const uint8_t* blk = row + (size_t)g * Q8_0_BYTES;
        const float d = f16_value((unsigned short)(blk[0] | (blk[1] << 8)));
        for (int l = 0; l < 32; ++l) dst[l] = from_float<T>((float)(int8_t)blk[2 + l] * d);
    } else if (type == TYPE_Q4_K) {
        const uint8_t* sb = row + (size_t)(g >> 3) * Q4_K_BYTES;
        const int j = g & 7;
        int sc, m;
        scale_min_k4(j, sb + 4, sc, m);
        const float d1 = f16_value((unsigned short)(sb[0] | (sb[1] << 8))) * (float)sc;
        const float m1 = f16_value((unsigned short)(sb[2] | (sb[3] << 8))) * (float)m;
        const uint8_t* q = sb + 16 + 32 * (j >> 1);
        for (int l = 0; l < 32; ++l) dst[l] = from_float<T>(d1 * (float)((j & 1) ? (q[l] >> 4) : (q[l] & 0xF)) - m1);
    } else {
        const uint8_t* sb = row + (size_t)(g >> 3) * Q6_K_BYTES;
        const int n = (g >> 2) & 1, qd = g & 3;
        const float d = f16_value((unsigned short)(sb[208] | (sb[209] << 8)));
        const uint8_t* ql = sb + 64 * n + 32 * (qd & 1);
        const uint8_t* qh = sb + 128 + 32 * n;
        const int8_t* sc = reinterpret_cast<const int8_t*>(sb + 192 + 8 * n + 2 * qd);
        for (int l = 0; l < 32; ++l) {
            const int lo = (qd & 2) ? (ql[l] >> 4) : (ql[l] & 0xF);
            const int q = (int)(int8_t)(lo | (((qh[l] >> (2 * qd)) & 3) << 4)) - 32;
            dst[l] = from_float<T>(d * (float)sc[l >> 4] * (float)q);
        }
    }
}

// rows == nullptr: row i of the output is row i of the matrix (to_float); else row ids[i] (get_rows)
template <typename T>
__global__ void __launch_bounds__(256) dequant_rows_kernel(int type, const uint8_t* __restrict__ w, const int* __restrict__ ids, T* __restrict__ out,
                                                           long long nrows_out, int K, long long nrows_w, unsigned int* status) {
    const long long groups_per_row = K / 32;
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nrows_out * groups_per_row) return;
    const long long r = i / groups_per_row;
    const int g = (int)(i - r * groups_per_row);
    long long src = ids != nullptr ? (long long)ids[r] : r;
    T* dst = out + r * K + (long long)g * 32;
    if (src < 0 || src >= nrows_w) {  // an id outside the table: zeros, and the status word says so
        for (int l = 0; l < 32; ++l) dst[l] = from_float<T>(0.0f);
        if (g == 0) record_failure(status, STATUS_BAD_ROW_ID, (unsigned int)r);
        return;
    }
    const size_t row_bytes = (size_t)(K / type_block_elems(type)) * type_block_bytes(type);
    dequant_group32<T>(type, w + (size_t)src * row_bytes, g, dst);
}

int quantize_weights(int type, const float* x, void* out, long long n, cudaStream_t s) {
    if (type_block_bytes(type) == 0) return B200Q_ERR_UNSUPPORTED;
    if (n < 0 || n % type_block_elems(type) != 0 || reinterpret_cast<uintptr_t>(out) % 2 != 0) return B200Q_ERR_INVALID;
    if (n == 0) return 0;
    const long long nb = n / type_block_elems(type);
    if (type == TYPE_Q8_0) quantize_q8_0_kernel<<<(unsigned)((nb + 255) / 256), 256, 0, s>>>(x, static_cast<uint8_t*>(out), nb);
    else if (type == TYPE_Q4_K) quantize_q4_k_kernel<<<(unsigned)((nb + 63) / 64), 64, 0, s>>>(x, static_cast<uint8_t*>(out), nb);
    else quantize_q6_k_kernel<<<(unsigned)((nb + 63) / 64), 64, 0, s>>>(x, static_cast<uint8_t*>(out), nb);
    return (int)cudaGetLastError();
}

int dequantize_rows(int type, int elem, const void* w, const int* ids, void* out, long long nrows_out, int K, long long nrows_w,
                    cudaStream_t s) {
    if (type_block_bytes(type) == 0) return B200Q_ERR_UNSUPPORTED;
    if (K <= 0 || K % type_block_elems(type) != 0 || nrows_out < 0 || nrows_w < 0) return B200Q_ERR_INVALID;
    if (nrows_out == 0) return 0;
    const long long threads = nrows_out * (K / 32);
    const unsigned grid = (unsigned)((threads + 255) / 256);
    const uint8_t* wp = static_cast<const uint8_t*>(w);
    if (elem == ELEM_F32) dequant_rows_kernel<float><<<grid, 256, 0, s>>>(type, wp, ids, static_cast<float*>(out), nrows_out, K, nrows_w, status_ptr());
    else if (elem == ELEM_F16) dequant_rows_kernel<__half><<<grid, 256, 0, s>>>(type, wp, ids, static_cast<__half*>(out), nrows_out, K, nrows_w, status_ptr());
    else if (elem == ELEM_BF16)
        dequant_rows_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(type, wp, ids, static_cast<__nv_bfloat16*>(out), nrows_out, K, nrows_w, status_ptr());
    else return B200Q_ERR_INVALID;
    return (int)cudaGetLastError();
}

}  // namespace b200q

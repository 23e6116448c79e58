// Q8_0 weights against UNQUANTIZED activations, accumulated in f32: the matvec the reference keeps for reads whose
// activations eight bits per 32 values would perturb too much (q8_0_exact_rows,
// crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_instance_q8_0.cu:14-96; launchers :98-140; host side
// fast_mmvq::exact, crates/inference-quant/src/gguf/fast_mmvq.rs:415-470). dst[b][row] = sum_k d(row, k/32) q(row, k) x[b][k]
// for 1..8 contiguous activation rows x [b][ncols] in bf16 or f32; dst [b][nrows] in the same type.
//
// HBM-bound on the weights like the decode GEMV, but the activations stay 16 / 32 bits wide, so the dot products are
// f32 FMAs instead of dp4a: a warp owns a weight row, lane l takes blocks l, l + 32, ... (a block is 34 bytes, 2-byte
// aligned: read as aligned words and funnel-shifted), activations come through L1 (every warp of every CTA reads the
// same few KB). Persistent grid of two CTAs per SM walking the rows.
#include "common.cuh"
#include "runtime.h"

namespace b200q {

constexpr int EXACT_WARPS = 8;

template <typename T> __device__ __forceinline__ void load_acts32(const T* p, float (&x)[32]);
template <> __device__ __forceinline__ void load_acts32<float>(const float* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
        x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
}
template <> __device__ __forceinline__ void load_acts32<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            // a bf16 is the upper half of an f32
            x[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
            x[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    }
}
// rows that are not 16-byte aligned (odd ncols multiples): element loads
template <typename T> __device__ __forceinline__ void load_acts32_slow(const T* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 32; ++i) x[i] = to_float<T>(p[i]);
}

template <typename T, int B>
__global__ void __launch_bounds__(EXACT_WARPS * 32) gemv_exact_q8_0_kernel(const uint8_t* __restrict__ w, const T* __restrict__ x,
                                                                          T* __restrict__ dst, int ncols, int nrows, int vec) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nblocks = ncols / QK8;
    const size_t row_bytes = (size_t)nblocks * Q8_0_BYTES;
    for (int row = blockIdx.x * EXACT_WARPS + warp; row < nrows; row += gridDim.x * EXACT_WARPS) {
        const uint8_t* wr = w + (size_t)row * row_bytes;
        float acc[B];
#pragma unroll
        for (int b = 0; b < B; ++b) acc[b] = 0.0f;
        for (int i = lane; i < nblocks; i += 32) {
            // 34 bytes at a 2-byte-aligned address: ten aligned words, shifted
            const uintptr_t a = reinterpret_cast<uintptr_t>(wr + (size_t)i * Q8_0_BYTES);
            const uint32_t shift = (uint32_t)(a & 2u) * 8u;
            const uint32_t* base = reinterpret_cast<const uint32_t*>(a & ~(uintptr_t)3);
            uint32_t raw[10], wd[9];
#pragma unroll
            for (int j = 0; j < 10; ++j) raw[j] = __ldg(base + j);
#pragma unroll
            for (int j = 0; j < 9; ++j) wd[j] = __funnelshift_r(raw[j], raw[j + 1], shift);
            const float d = half_bits_to_float(wd[0]);
            float wv[32];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint32_t q = __funnelshift_r(wd[j], wd[j + 1], 16);  // quants 4j .. 4j+3
                wv[4 * j] = d * (float)(int)(int8_t)(q & 0xffu);
                wv[4 * j + 1] = d * (float)(int)(int8_t)((q >> 8) & 0xffu);
                wv[4 * j + 2] = d * (float)(int)(int8_t)((q >> 16) & 0xffu);
                wv[4 * j + 3] = d * (float)(int)(int8_t)(q >> 24);
            }
#pragma unroll
            for (int b = 0; b < B; ++b) {
                float xv[32];
                const T* xp = x + (size_t)b * ncols + (size_t)i * QK8;
                if (vec) load_acts32<T>(xp, xv);
                else load_acts32_slow<T>(xp, xv);
                float s = 0.0f;
#pragma unroll
                for (int j = 0; j < 32; ++j) s = fmaf(wv[j], xv[j], s);
                acc[b] += s;
            }
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const float v = warp_sum(acc[b]);
            if (lane == 0) dst[(size_t)b * nrows + row] = from_float<T>(v);
        }
    }
}

template <typename T>
static int launch_exact(const void* vx, const void* vy, void* dst, int ncols, int nrows, int b, cudaStream_t s) {
    if (ncols <= 0 || nrows <= 0 || ncols % QK8 != 0 || b < 1) return b < 1 ? B200Q_ERR_INVALID : 0;
    if (b > 8) b = 8;  // the reference's launcher clamps the same way (its switch's default case)
    if (reinterpret_cast<uintptr_t>(vx) % 2 != 0) return B200Q_ERR_UNSUPPORTED;
    const int vec = (reinterpret_cast<uintptr_t>(vy) % 16 == 0) && (((size_t)ncols * sizeof(T)) % 16 == 0);
    const int ctas_needed = (nrows + EXACT_WARPS - 1) / EXACT_WARPS;
    const int grid = ctas_needed < 4 * runtime_info().sm_count ? ctas_needed : 4 * runtime_info().sm_count;
    const uint8_t* w = static_cast<const uint8_t*>(vx);
    const T* x = static_cast<const T*>(vy);
    T* d = static_cast<T*>(dst);
    switch (b) {
#define B200Q_EXACT_CASE(BB) \
    case BB: gemv_exact_q8_0_kernel<T, BB><<<grid, EXACT_WARPS * 32, 0, s>>>(w, x, d, ncols, nrows, vec); break;
        B200Q_EXACT_CASE(1) B200Q_EXACT_CASE(2) B200Q_EXACT_CASE(3) B200Q_EXACT_CASE(4)
        B200Q_EXACT_CASE(5) B200Q_EXACT_CASE(6) B200Q_EXACT_CASE(7) B200Q_EXACT_CASE(8)
#undef B200Q_EXACT_CASE
    }
    return (int)cudaGetLastError();
}

}  // namespace b200q

// The reference's symbols (crates/inference-quant/src/gguf/ffi.rs:1004-1021); void, asynchronous, allocation-free.
extern "C" void launch_mmvq_gguf_q8_0_bf16_exact(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int b_size,
                                                 void* stream) {
    b200q::note_launch_status(b200q::launch_exact<__nv_bfloat16>(vx, vy, dst, ncols_x, nrows_x, b_size, (cudaStream_t)stream));
}
extern "C" void launch_mmvq_gguf_q8_0_f32_exact(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int b_size,
                                                void* stream) {
    b200q::note_launch_status(b200q::launch_exact<float>(vx, vy, dst, ncols_x, nrows_x, b_size, (cudaStream_t)stream));
}

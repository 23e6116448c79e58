// Activation quantizers of the GGUF matmul path.
//
//  * decode: rows of bf16/f16/f32 -> Q8_1 blocks {f16 d; f16 sum(x); i8 qs[32]}, rows padded with zeros to
//    kx_padded. Same values as the reference kernel `mmvq_gguf_quantize_q8_1_*`
//    (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_quantize.cu:9-107): d = amax / 127,
//    q = roundf(x / d), sum = 32-lane xor butterfly of x. Divisions are IEEE here.
//  * prefill: rows -> 144-byte blocks of 128 values in the column-of-blocks order of
//    `quantize_mmq_q8_1` (crates/inference-quant/kernels/cuda/mmq_gguf/mmq_quantize.cu:98-199):
//    d_inv = 127 / amax, q = roundf(x * d_inv), d = 1 / d_inv; D4 stores float d, DS4 half2 (d, sum(x)).
#include "common.cuh"

namespace b200q {

// One warp per 32-value block; 8 warps per CTA; grid-stride over blocks.
template <typename src_t>
__global__ void __launch_bounds__(256) quantize_q8_1_kernel(const src_t* __restrict__ x, uint8_t* __restrict__ vy,
                                                            int kx, int kx_padded, int num_rows) {
    grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const int blocks_per_row = kx_padded / 32;
    const long long total = (long long)blocks_per_row * num_rows;
    for (long long blk = (long long)blockIdx.x * 8 + (threadIdx.x >> 5); blk < total; blk += (long long)gridDim.x * 8) {
        const int row = (int)(blk / blocks_per_row);
        const int kb = (int)(blk - (long long)row * blocks_per_row);
        const int ix = kb * 32 + lane;
        const float xi = ix < kx ? to_float<src_t>(x[(long long)row * kx + ix]) : 0.0f;
        const float amax = warp_max(fabsf(xi));
        const float sum = warp_sum(xi);
        const float d = amax / 127.0f;
        const int q = amax == 0.0f ? 0 : (int)roundf(xi / d);
        uint8_t* yb = vy + blk * Q8_1_BYTES;
        reinterpret_cast<int8_t*>(yb + 4)[lane] = (int8_t)q;
        if (lane == 0) {
            __half2 ds = __halves2half2(__float2half_rn(d), __float2half_rn(sum));
            *reinterpret_cast<__half2*>(yb) = ds;
        }
    }
    grid_launch_dependents();
}

template <typename src_t>
static void launch_quantize_q8_1(const void* x, void* vy, int kx, int kx_padded, int num_rows, cudaStream_t s) {
    if (num_rows <= 0 || kx_padded <= 0) return;
    const long long total = (long long)(kx_padded / 32) * num_rows;
    long long ctas = (total + 7) / 8;
    if (ctas > 148 * 8) ctas = 148 * 8;
    quantize_q8_1_kernel<src_t><<<(unsigned)ctas, 256, 0, s>>>((const src_t*)x, (uint8_t*)vy, kx, kx_padded, num_rows);
}

// ---------------------------------------------------------------------------------------------
// prefill layout. Each thread holds 4 consecutive values; 8 threads a 32-value group.
// ---------------------------------------------------------------------------------------------
enum MmqLayout : int { MMQ_D4 = 0, MMQ_DS4 = 1 };

template <typename src_t>
__device__ __forceinline__ float4 load4(const src_t* x, long long base, long long i0, long long ne00) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i0 + 0 < ne00) v.x = to_float<src_t>(x[base + 0]);
    if (i0 + 1 < ne00) v.y = to_float<src_t>(x[base + 1]);
    if (i0 + 2 < ne00) v.z = to_float<src_t>(x[base + 2]);
    if (i0 + 3 < ne00) v.w = to_float<src_t>(x[base + 3]);
    return v;
}

// act(gate) * up as the reference's fused quantizer forms it (kernels/cuda/mmq_gguf/mmq_quantize.cu:201-235): the
// activation in f32, rounded to the input type, the product in the input type. Activation ids: 0 SiLU, 1 GELU (tanh),
// 2 ReLU, 3 GELU (erf), 4 sigmoid; anything else SiLU.
__device__ __forceinline__ float mmq_glu_act(float x, int act) {
    switch (act) {
        case 1: return 0.5f * x * (1.0f + tanhf(0.7978845608f * (x + 0.044715f * (x * x * x))));
        case 2: return fmaxf(x, 0.0f);
        case 3: return x * normcdff(x);
        case 4: return 1.0f / (1.0f + expf(-x));
        default: return x / (1.0f + expf(-x));
    }
}
template <typename src_t> __device__ __forceinline__ float mmq_glu_product(float gate, float up, int act) {
    if constexpr (sizeof(src_t) == 4) return mmq_glu_act(gate, act) * up;
    else return to_float<src_t>(__hmul(from_float<src_t>(mmq_glu_act(gate, act)), from_float<src_t>(up)));
}

// grid (rows, ceil(ne0 / 512)), block 128: thread t of block (row, cy) takes values i0 = (128 cy + t) * 4.
// GLU: x is the gate, `up` the second operand of the same shape, and act(gate) * up is what gets quantized
// (launch_mmq_quantize_glu_q8_1_*: the MLP's down projection reads its prefill activations straight from gate and up).
template <typename src_t, int LAYOUT, bool GLU = false>
__global__ void __launch_bounds__(128) quantize_mmq_q8_1_kernel(const src_t* __restrict__ x, const int32_t* __restrict__ ids,
                                                               uint8_t* __restrict__ vy, long long ne00, long long s01,
                                                               long long ne0, int ne1, const src_t* __restrict__ up = nullptr,
                                                               int activation = 0) {
    grid_dependency_wait();
    const long long i0 = ((long long)blockDim.x * blockIdx.y + threadIdx.x) * 4;
    // ne0 is a multiple of 128, so a warp (128 values) is inside or outside as a whole and the shuffles below
    // always see all 32 lanes
    if (i0 < ne0) {
        const long long i1 = blockIdx.x;
        const long long i01 = ids ? ids[i1] : i1;
        const long long ib = (i0 / 128) * ne1 + i1;
        const int iqs = (int)(i0 % 128);
        float4 xi = load4<src_t>(x, i01 * s01 + i0, i0, ne00);
        if constexpr (GLU) {
            const float4 u = load4<src_t>(up, i01 * s01 + i0, i0, ne00);
            xi = make_float4(mmq_glu_product<src_t>(xi.x, u.x, activation), mmq_glu_product<src_t>(xi.y, u.y, activation),
                             mmq_glu_product<src_t>(xi.z, u.z, activation), mmq_glu_product<src_t>(xi.w, u.w, activation));
        }
        float amax = fmaxf(fmaxf(fabsf(xi.x), fabsf(xi.y)), fmaxf(fabsf(xi.z), fabsf(xi.w)));
#pragma unroll
        for (int off = 4; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        float sum = 0.0f;
        if (LAYOUT == MMQ_DS4) {
            sum = xi.x + xi.y + xi.z + xi.w;
#pragma unroll
            for (int off = 4; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
        }
        const float d_inv = 127.0f / amax;
        char4 q;
        q.x = amax == 0.0f ? 0 : (signed char)roundf(xi.x * d_inv);
        q.y = amax == 0.0f ? 0 : (signed char)roundf(xi.y * d_inv);
        q.z = amax == 0.0f ? 0 : (signed char)roundf(xi.z * d_inv);
        q.w = amax == 0.0f ? 0 : (signed char)roundf(xi.w * d_inv);
        uint8_t* blk = vy + ib * MMQ_BLOCK_BYTES;
        reinterpret_cast<char4*>(blk + 16)[iqs / 4] = q;
        if (iqs % 32 == 0) {
            const float d = amax == 0.0f ? 0.0f : 1.0f / d_inv;
            if (LAYOUT == MMQ_DS4) {
                reinterpret_cast<__half2*>(blk)[iqs / 32] = __halves2half2(__float2half_rn(d), __float2half_rn(sum));
            } else {
                reinterpret_cast<float*>(blk)[iqs / 32] = d;
            }
        }
    }
    grid_launch_dependents();
}

template <int LAYOUT>
static void launch_quantize_mmq(const void* x, const int32_t* ids, void* vy, int type_x, long long ne00, long long s01,
                                long long ne0, long long ne1, cudaStream_t s) {
    if (ne1 <= 0 || ne0 <= 0) return;
    dim3 grid((unsigned)ne1, (unsigned)((ne0 + 511) / 512), 1);
    // type_x follows the reference: 0 = f32, 1 = f16, 30 = bf16 (crates/inference-quant/src/gguf/fast_mmq.rs:671-676)
    if (type_x == 0)
        quantize_mmq_q8_1_kernel<float, LAYOUT><<<grid, 128, 0, s>>>((const float*)x, ids, (uint8_t*)vy, ne00, s01, ne0, (int)ne1);
    else if (type_x == 1)
        quantize_mmq_q8_1_kernel<__half, LAYOUT><<<grid, 128, 0, s>>>((const __half*)x, ids, (uint8_t*)vy, ne00, s01, ne0, (int)ne1);
    else
        quantize_mmq_q8_1_kernel<__nv_bfloat16, LAYOUT><<<grid, 128, 0, s>>>((const __nv_bfloat16*)x, ids, (uint8_t*)vy, ne00, s01, ne0, (int)ne1);
}

template <int LAYOUT>
static void launch_quantize_mmq_glu(const void* gate, const void* up, const int32_t* ids, void* vy, int type_x, long long ne00,
                                    long long s01, long long ne0, long long ne1, int activation, cudaStream_t s) {
    if (ne1 <= 0 || ne0 <= 0) return;
    dim3 grid((unsigned)ne1, (unsigned)((ne0 + 511) / 512), 1);
    if (type_x == 0)
        quantize_mmq_q8_1_kernel<float, LAYOUT, true><<<grid, 128, 0, s>>>((const float*)gate, ids, (uint8_t*)vy, ne00, s01, ne0, (int)ne1,
                                                                          (const float*)up, activation);
    else if (type_x == 1)
        quantize_mmq_q8_1_kernel<__half, LAYOUT, true><<<grid, 128, 0, s>>>((const __half*)gate, ids, (uint8_t*)vy, ne00, s01, ne0, (int)ne1,
                                                                           (const __half*)up, activation);
    else
        quantize_mmq_q8_1_kernel<__nv_bfloat16, LAYOUT, true><<<grid, 128, 0, s>>>((const __nv_bfloat16*)gate, ids, (uint8_t*)vy, ne00, s01, ne0,
                                                                                  (int)ne1, (const __nv_bfloat16*)up, activation);
}

}  // namespace b200q

using namespace b200q;

extern "C" {

void launch_mmvq_gguf_quantize_q8_1_bf16(const void* x, void* vy, int kx, int kx_padded, int num_rows, void* stream) {
    launch_quantize_q8_1<__nv_bfloat16>(x, vy, kx, kx_padded, num_rows, (cudaStream_t)stream);
}
void launch_mmvq_gguf_quantize_q8_1_f16(const void* x, void* vy, int kx, int kx_padded, int num_rows, void* stream) {
    launch_quantize_q8_1<__half>(x, vy, kx, kx_padded, num_rows, (cudaStream_t)stream);
}
void launch_mmvq_gguf_quantize_q8_1_f32(const void* x, void* vy, int kx, int kx_padded, int num_rows, void* stream) {
    launch_quantize_q8_1<float>(x, vy, kx, kx_padded, num_rows, (cudaStream_t)stream);
}

// Only the 2-D case the dense matmul path uses (ne2 = ne3 = 1) is implemented; s02/s03 are accepted and unused.
void launch_mmq_quantize_q8_1_D4(const void* x, const int32_t* ids, void* vy, int type_x, int64_t ne00, int64_t s01,
                                 int64_t s02, int64_t s03, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3,
                                 void* stream) {
    (void)s02; (void)s03; (void)ne2; (void)ne3;
    launch_quantize_mmq<MMQ_D4>(x, ids, vy, type_x, ne00, s01, ne0, ne1, (cudaStream_t)stream);
}
void launch_mmq_quantize_q8_1_DS4(const void* x, const int32_t* ids, void* vy, int type_x, int64_t ne00, int64_t s01,
                                  int64_t s02, int64_t s03, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3,
                                  void* stream) {
    (void)s02; (void)s03; (void)ne2; (void)ne3;
    launch_quantize_mmq<MMQ_DS4>(x, ids, vy, type_x, ne00, s01, ne0, ne1, (cudaStream_t)stream);
}

// The prefill quantizer with the gated activation folded in: act(gate) * up, rows of ne00 values at stride s01, quantized to
// the same blocks as launch_mmq_quantize_q8_1_* (crates/inference-quant/src/gguf/ffi.rs:702-770).
void launch_mmq_quantize_glu_q8_1_D4(const void* gate, const void* up, const int32_t* ids, void* vy, int type_x, int64_t ne00, int64_t s01,
                                     int64_t ne0, int64_t ne1, int activation, void* stream) {
    launch_quantize_mmq_glu<MMQ_D4>(gate, up, ids, vy, type_x, ne00, s01, ne0, ne1, activation, (cudaStream_t)stream);
}
void launch_mmq_quantize_glu_q8_1_DS4(const void* gate, const void* up, const int32_t* ids, void* vy, int type_x, int64_t ne00, int64_t s01,
                                      int64_t ne0, int64_t ne1, int activation, void* stream) {
    launch_quantize_mmq_glu<MMQ_DS4>(gate, up, ids, vy, type_x, ne00, s01, ne0, ne1, activation, (cudaStream_t)stream);
}
void launch_mmq_quantize_glu_q8_1_D4_f32(const float* gate, const float* up, const int32_t* ids, void* vy, int64_t ne00, int64_t s01,
                                         int64_t ne0, int64_t ne1, int activation, void* stream) {
    launch_quantize_mmq_glu<MMQ_D4>(gate, up, ids, vy, 0, ne00, s01, ne0, ne1, activation, (cudaStream_t)stream);
}
void launch_mmq_quantize_glu_q8_1_DS4_f32(const float* gate, const float* up, const int32_t* ids, void* vy, int64_t ne00, int64_t s01,
                                          int64_t ne0, int64_t ne1, int activation, void* stream) {
    launch_quantize_mmq_glu<MMQ_DS4>(gate, up, ids, vy, 0, ne00, s01, ne0, ne1, activation, (cudaStream_t)stream);
}

}  // extern "C"

// Decode GEMV for callers that must not allocate device memory.
//
// The two-launch decode path needs a scratch buffer for the Q8_1 activation blocks between the quantize launch and
// the GEMV launch, and normally the caller allocates it. Some callers cannot: a serving loop whose device memory is
// entirely owned by its own pool, a thread that may not call cudaMalloc because cudaMalloc synchronizes the whole
// device and would stall the other streams, or code that runs where an allocation failure cannot be handled. For
// them this file keeps the scratch in a fixed array that is part of the library image itself: every GPU that loads
// the library reserves B200Q_STATIC_SCRATCH_BYTES for it until the process exits, and nothing is ever allocated or
// freed here.
#include <cstdio>

#include "common.cuh"
#include "runtime.h"

extern "C" {
void launch_mmvq_gguf_quantize_q8_1_bf16(const void*, void*, int, int, int, void*);
void launch_mmvq_gguf_quantize_q8_1_f16(const void*, void*, int, int, int, void*);
void launch_mmvq_gguf_quantize_q8_1_f32(const void*, void*, int, int, int, void*);
}

namespace b200q {
struct PeerExchange;
int gemv_q4_k(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
int gemv_q6_k(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
int gemv_q8_0(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
int set_error(int code, const char* msg);

// Largest problem the fixed scratch holds: 8 activation rows of 32768 values (padded), 36 bytes per 32 values.
constexpr int STATIC_MAX_ROWS = 8;
constexpr int STATIC_MAX_K_PADDED = 32768;
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)STATIC_MAX_ROWS * (STATIC_MAX_K_PADDED / 32) * Q8_1_BYTES;  // 294,912

// In host code this name is only a handle for the runtime; the device address comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_q8_1_scratch[STATIC_SCRATCH_BYTES];

// Device address of the scratch array on the current device, looked up once per device.
static int static_scratch_ptr(void** out) {
    static void* cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return B200Q_ERR_INVALID;
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_q8_1_scratch);
        if (e != cudaSuccess) return (int)e;
        cached[dev] = p;
    }
    *out = cached[dev];
    return 0;
}
}  // namespace b200q

using namespace b200q;

// Quantize x to Q8_1 blocks in the library's fixed scratch array, then run the decode GEMV on them: the same two
// kernels, in the same order, as launch_mmvq_gguf_quantize_q8_1_<elem> followed by launch_mmvq_gguf_<type>_<elem>_plain,
// so the output is identical to that pair's. Nothing is allocated.
extern "C" int b200q_gemv_static_scratch(int type, int elem, const void* w, const void* x, void* dst, int K, int N,
                                         int stride_dst, int b_size, void* stream) {
    if (!w || !x || !dst) return set_error(B200Q_ERR_INVALID, "null pointer");
    if (type_block_bytes(type) == 0) return set_error(B200Q_ERR_UNSUPPORTED, "weight type is not Q8_0, Q4_K or Q6_K");
    if (elem != ELEM_F32 && elem != ELEM_F16 && elem != ELEM_BF16) return set_error(B200Q_ERR_INVALID, "bad element type");
    if (K <= 0 || K % type_block_elems(type) != 0) return set_error(B200Q_ERR_INVALID, "K is not a multiple of the block size");
    const int k_padded = (K + 511) / 512 * 512;
    if (b_size < 1 || b_size > STATIC_MAX_ROWS || k_padded > STATIC_MAX_K_PADDED) {
        static thread_local char msg[160];
        std::snprintf(msg, sizeof msg,
                      "b200q_gemv_static_scratch holds at most %d activation rows of %d values (%zu bytes); got %d rows of %d",
                      STATIC_MAX_ROWS, STATIC_MAX_K_PADDED, STATIC_SCRATCH_BYTES, b_size, K);
        return set_error(B200Q_ERR_TOO_LARGE, msg);
    }
    void* scratch = nullptr;
    const int rc0 = static_scratch_ptr(&scratch);
    if (rc0 != 0) return set_error(rc0, rc0 > 0 ? cudaGetErrorString((cudaError_t)rc0) : "no device for the static scratch");
    // every block of the padded rows is rewritten by the quantizer (padding as zeros), so nothing left over from an
    // earlier call is ever read
    if (elem == ELEM_BF16) launch_mmvq_gguf_quantize_q8_1_bf16(x, scratch, K, k_padded, b_size, stream);
    else if (elem == ELEM_F16) launch_mmvq_gguf_quantize_q8_1_f16(x, scratch, K, k_padded, b_size, stream);
    else launch_mmvq_gguf_quantize_q8_1_f32(x, scratch, K, k_padded, b_size, stream);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error((int)e, cudaGetErrorString(e));
    int rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (type == TYPE_Q4_K) rc = gemv_q4_k(elem, w, scratch, dst, K, N, k_padded / 32, stride_dst, b_size, 0, nullptr, s);
    else if (type == TYPE_Q6_K) rc = gemv_q6_k(elem, w, scratch, dst, K, N, k_padded / 32, stride_dst, b_size, 0, nullptr, s);
    else rc = gemv_q8_0(elem, w, scratch, dst, K, N, k_padded / 32, stride_dst, b_size, 0, nullptr, s);
    take_launch_status();
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "gemv failed");
    return B200Q_OK;
}

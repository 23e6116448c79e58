/*
 * C ABI of libinferencequant_b200.so: sm_100a kernels for the GGUF quantized-weight matmul path
 * (Q8_0 / Q4_K / Q6_K weights in their unchanged GGUF block layout).
 *
 * Part 1 re-exports, with identical names and argument lists, the `extern "C"` launchers the reference
 * resolves with dlopen from `libinferencequant[_<type>].so` (crates/inference-tensor/src/kernel_library.rs:244-393,
 * declarations in crates/inference-quant/src/gguf/ffi.rs). All pointers are DEVICE pointers owned by the caller,
 * `stream` is a CUstream passed as void*, every launcher is asynchronous on that stream, allocates nothing, never
 * synchronizes and returns nothing; `int` is 32 bits.
 *
 * Part 2 is this library's own status-returning API: 0 = ok, > 0 = a cudaError_t, < 0 = a B200Q_ERR_* code,
 * with a thread-local message from b200q_last_error().
 */
#ifndef INFERENCEQUANT_B200_H
#define INFERENCEQUANT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------------------------------
 * Part 1: the reference's launcher symbols
 * ------------------------------------------------------------------------------------------------------------ */

/* Loader handshake: the host refuses a library whose id differs from the one compiled into it
 * (crates/inference-tensor/src/kernel_library.rs:8,288-297). */
extern const char inference_kernel_build_id[];

/* Activation rows -> Q8_1 blocks {f16 d; f16 sum(x); i8 qs[32]} (36 bytes per 32 values), each row padded with
 * zeros from kx to kx_padded (a multiple of 32; the reference passes pad(kx, 512)). vy holds
 * num_rows * kx_padded / 32 blocks. d = amax / 127, q = roundf(x / d).
 * Replaces crates/inference-quant/src/gguf/ffi.rs:602-629 (kernel: kernels/cuda/mmvq_gguf/mmvq_quantize.cu:9-146). */
void launch_mmvq_gguf_quantize_q8_1_bf16(const void* x, void* vy, int kx, int kx_padded, int num_rows, void* stream);
void launch_mmvq_gguf_quantize_q8_1_f16(const void* x, void* vy, int kx, int kx_padded, int num_rows, void* stream);
void launch_mmvq_gguf_quantize_q8_1_f32(const void* x, void* vy, int kx, int kx_padded, int num_rows, void* stream);

/* Decode GEMV: dst[j * stride_col_dst + row] = sum_k W[row][k] * y[j][k] for j < b_size (1..8).
 * vx: packed weights [nrows_x][ncols_x / block] blocks, rows contiguous; vy: Q8_1 blocks, row j at block
 * j * stride_col_y; dst element type is the name's suffix.
 * Replaces crates/inference-quant/src/gguf/ffi.rs:846-878 (kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:688-759,1762-1834).
 * The fast path needs vx 16-byte aligned with at least 16 readable bytes after the last block (the reference's
 * device buffers carry 512 elements' worth of padding, crates/inference-tensor/src/quantized/cuda.rs:511-530) and
 * ncols_x a multiple of 64; other inputs take a slower kernel. */
void launch_mmvq_gguf_q8_0_bf16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                      int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q8_0_f16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                     int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q8_0_f32_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                     int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q4_k_bf16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                      int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q4_k_f16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                     int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q4_k_f32_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                     int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q6_k_bf16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                      int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q6_k_f16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                     int stride_col_y, int stride_col_dst, int b_size, void* stream);
void launch_mmvq_gguf_q6_k_f32_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x,
                                     int stride_col_y, int stride_col_dst, int b_size, void* stream);

/* Small-batch tensor-core matvec, as the reference's host drives it (fast_mmvq::tiled_plain,
 * crates/inference-quant/src/gguf/fast_mmvq.rs:2049-2126): launch_mmvq_tc_quantize_<elem> lays num_rows (1..16) rows
 * x [num_rows][kx] out in the tier's activation format - the rows in halves of 8, per half and 32-value block 32 int2
 * fragments, then the 8 rows' f16 scales, then their int16 sums: 288 bytes per block and half, the host's scratch
 * (fast_mmvq.rs:94,1898-1902) - and launch_mmvq_tc_gguf_<type>_<elem>_plain computes
 * dst[j * stride_col_dst + row] = sum_k W[row][k] * x[j][k] for j < b_size from it. `cfg` picks among the reference
 * kernel's own launch shapes and is ignored here. Needs ncols_x a multiple of 256.
 * Replaces crates/inference-quant/src/gguf/ffi.rs:631-652,954-998 (kernels/cuda/mmvq_gguf/mmvq_quantize.cu:148-190,
 * mmvq_tc_k.cuh:221-388). */
void launch_mmvq_tc_quantize_bf16(const void* x, void* vy, int kx, int num_rows, void* stream);
void launch_mmvq_tc_quantize_f16(const void* x, void* vy, int kx, int num_rows, void* stream);
void launch_mmvq_tc_quantize_f32(const void* x, void* vy, int kx, int num_rows, void* stream);
void launch_mmvq_tc_gguf_q4_k_bf16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int stride_col_dst,
                                         int b_size, int cfg, void* stream);
void launch_mmvq_tc_gguf_q4_k_f16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int stride_col_dst,
                                        int b_size, int cfg, void* stream);
void launch_mmvq_tc_gguf_q4_k_f32_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int stride_col_dst,
                                        int b_size, int cfg, void* stream);
void launch_mmvq_tc_gguf_q6_k_bf16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int stride_col_dst,
                                         int b_size, int cfg, void* stream);
void launch_mmvq_tc_gguf_q6_k_f16_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int stride_col_dst,
                                        int b_size, int cfg, void* stream);
void launch_mmvq_tc_gguf_q6_k_f32_plain(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int stride_col_dst,
                                        int b_size, int cfg, void* stream);

/* Q8_0 weights against UNQUANTIZED activations, f32 accumulation: dst[j * nrows_x + row] = sum_k W[row][k] * y[j][k],
 * y [b_size][ncols_x] contiguous rows and dst [b_size][nrows_x], both of the suffix's type; b_size 1..8 (larger values
 * are treated as 8, as the reference's launcher does).
 * Replaces crates/inference-quant/src/gguf/ffi.rs:1004-1021 (kernels/cuda/mmvq_gguf/mmvq_instance_q8_0.cu:14-140). */
void launch_mmvq_gguf_q8_0_bf16_exact(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int b_size,
                                      void* stream);
void launch_mmvq_gguf_q8_0_f32_exact(const void* vx, const void* vy, void* dst, int ncols_x, int nrows_x, int b_size,
                                     void* stream);

/* Fused decode matvecs on Q8_1 activation blocks (vy as launch_mmvq_gguf_quantize_q8_1_* writes them, stride_col_y
 * blocks per activation row), b_size 1..8.
 *  fused_glu: dst[j * stride_col_dst + row] = act(gate[row] . y[j]) * (up[row] . y[j]) for two matrices of the same type
 *    and shape; gate and up are rounded to the output type, the activation is evaluated in f32 on the rounded gate and
 *    rounded, the product is formed in the output type. activation: 0 SiLU, 1 GELU (tanh), 2 ReLU, 3 GELU (erf),
 *    4 sigmoid; other ids mean SiLU.
 *  fused_qkv: three matrices of one type on the same activations: q_dst[j * nrows_q + row], k_dst[j * nrows_k + row],
 *    v_dst[j * nrows_v + row].
 * Replaces crates/inference-quant/src/gguf/ffi.rs:1032-1118 (kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:761-962; host side
 * fast_mmvq::fused_glu / fused_qkv). */
void launch_mmvq_gguf_q8_0_bf16_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                          int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                          void* stream);
void launch_mmvq_gguf_q8_0_f16_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                         int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                         void* stream);
void launch_mmvq_gguf_q8_0_f32_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                         int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                         void* stream);
void launch_mmvq_gguf_q4_k_bf16_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                          int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                          void* stream);
void launch_mmvq_gguf_q4_k_f16_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                         int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                         void* stream);
void launch_mmvq_gguf_q4_k_f32_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                         int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                         void* stream);
void launch_mmvq_gguf_q6_k_bf16_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                          int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                          void* stream);
void launch_mmvq_gguf_q6_k_f16_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                         int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                         void* stream);
void launch_mmvq_gguf_q6_k_f32_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst, int ncols_x,
                                         int nrows_x, int stride_col_y, int stride_col_dst, int b_size, int activation,
                                         void* stream);
void launch_mmvq_gguf_q8_0_bf16_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                          void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                          int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q8_0_f16_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                         void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                         int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q8_0_f32_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                         void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                         int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q4_k_bf16_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                          void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                          int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q4_k_f16_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                         void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                         int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q4_k_f32_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                         void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                         int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q6_k_bf16_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                          void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                          int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q6_k_f16_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                         void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                         int stride_col_y, int b_size, void* stream);
void launch_mmvq_gguf_q6_k_f32_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy, void* q_dst,
                                         void* k_dst, void* v_dst, int ncols_x, int nrows_q, int nrows_k, int nrows_v,
                                         int stride_col_y, int b_size, void* stream);

/* Prefill activation quantizer: rows -> 144-byte blocks of 128 values, block index (k / 128) * ne1 + row.
 * D4 stores four f32 scales, DS4 four half2 (d, sum(x)). type_x: 0 = f32, 1 = f16, 30 = bf16. ne00 = row length,
 * s01 = row stride in elements, ne0 = padded row length (multiple of 128), ne1 = rows; only ne2 = ne3 = 1.
 * Replaces crates/inference-quant/src/gguf/ffi.rs:657-685 (kernels/cuda/mmq_gguf/mmq_quantize.cu:98-199). */
void launch_mmq_quantize_q8_1_D4(const void* x, const int32_t* ids, void* vy, int type_x, int64_t ne00, int64_t s01,
                                 int64_t s02, int64_t s03, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3,
                                 void* stream);
void launch_mmq_quantize_q8_1_DS4(const void* x, const int32_t* ids, void* vy, int type_x, int64_t ne00, int64_t s01,
                                  int64_t s02, int64_t s03, int64_t ne0, int64_t ne1, int64_t ne2, int64_t ne3,
                                  void* stream);

/* The same quantizer with the gated activation of an MLP folded in: what is quantized is act(gate) * up (the activation
 * in f32, rounded to the input type; the product in the input type), so that the down projection's prefill activations
 * come straight from the gate and up outputs. gate, up: rows of ne00 values at stride s01; activation ids as for
 * fused_glu above. The _f32 forms take f32 inputs without a type argument.
 * Replaces crates/inference-quant/src/gguf/ffi.rs:702-770 (kernels/cuda/mmq_gguf/mmq_quantize.cu:201-330). */
void launch_mmq_quantize_glu_q8_1_D4(const void* gate, const void* up, const int32_t* ids, void* vy, int type_x, int64_t ne00,
                                     int64_t s01, int64_t ne0, int64_t ne1, int activation, void* stream);
void launch_mmq_quantize_glu_q8_1_DS4(const void* gate, const void* up, const int32_t* ids, void* vy, int type_x, int64_t ne00,
                                      int64_t s01, int64_t ne0, int64_t ne1, int activation, void* stream);
void launch_mmq_quantize_glu_q8_1_D4_f32(const float* gate, const float* up, const int32_t* ids, void* vy, int64_t ne00,
                                         int64_t s01, int64_t ne0, int64_t ne1, int activation, void* stream);
void launch_mmq_quantize_glu_q8_1_DS4_f32(const float* gate, const float* up, const int32_t* ids, void* vy, int64_t ne00,
                                          int64_t s01, int64_t ne0, int64_t ne1, int activation, void* stream);

/* Prefill matmul on activations quantized by launch_mmq_quantize_q8_1_{D4,DS4}: dst[token * stride_col_dst + row] =
 * sum_k W[row][k] * (d q)[token][k] for token < ncols_y, row < nrows_x. x: packed weights, stride_row_x blocks per row;
 * y: the 144-byte activation blocks (D4 for Q8_0 and Q6_K weights, DS4 for Q4_K: the reference's host pairs them so,
 * crates/inference-quant/src/gguf/fast_mmq.rs:167-190); type_dst: 0 = f32, 1 = f16, 30 = bf16. tmp_fixup (the
 * reference kernel's stream-k scratch), cc, nsm, smpbo and warp_size are accepted and not used. On tcgen05 tensor
 * cores when ncols_x is a multiple of 256 and the packed rows are 16-byte aligned, a plain kernel otherwise.
 * Replaces crates/inference-quant/src/gguf/ffi.rs:911-927 (kernels/cuda/mmq_gguf/mmq_gguf.cuh:3632-3875, host side
 * fast_mmq.rs:489-512). */
void launch_mmq_gguf_q8_0(void* tmp_fixup, const void* x, const void* y, void* dst, int64_t ncols_x, int64_t nrows_x,
                          int64_t ncols_y, int64_t stride_row_x, int64_t stride_col_dst, int cc, int nsm, int64_t smpbo,
                          int warp_size, int type_dst, void* stream);
void launch_mmq_gguf_q4_k(void* tmp_fixup, const void* x, const void* y, void* dst, int64_t ncols_x, int64_t nrows_x,
                          int64_t ncols_y, int64_t stride_row_x, int64_t stride_col_dst, int cc, int nsm, int64_t smpbo,
                          int warp_size, int type_dst, void* stream);
void launch_mmq_gguf_q6_k(void* tmp_fixup, const void* x, const void* y, void* dst, int64_t ncols_x, int64_t nrows_x,
                          int64_t ncols_y, int64_t stride_row_x, int64_t stride_col_dst, int cc, int nsm, int64_t smpbo,
                          int warp_size, int type_dst, void* stream);

/* ------------------------------------------------------------------------------------------------------------
 * Part 2: status-returning API
 * ------------------------------------------------------------------------------------------------------------ */

#define B200Q_OK 0
#define B200Q_ERR_UNSUPPORTED (-1)   /* no kernel for this shape / type / alignment */
#define B200Q_ERR_INVALID (-2)       /* bad argument */
#define B200Q_ERR_DEVICE_STATUS (-3) /* a kernel recorded a failure in the device status word */
#define B200Q_ERR_TOO_LARGE (-4)     /* beyond a fixed capacity */

/* GGUF type ids (crates/inference-tensor/src/quantized/mod.rs:582-624) */
#define B200Q_TYPE_Q8_0 8
#define B200Q_TYPE_Q4_K 12
#define B200Q_TYPE_Q6_K 14
/* element types */
#define B200Q_F32 0
#define B200Q_F16 1
#define B200Q_BF16 2

const char* b200q_version(void);
const char* b200q_last_error(void);

/* Options: "pdl" (launch GEMVs and quantizers with programmatic stream serialization), "force_simple_gemv",
 * "gemv_stage_bytes", "gemv_passes" (0 = the planner's choice, 1 or 2 passes of all warps per stage),
 * "gemv_pass_limit_bytes" (bytes one pass may cover before a row is given more warps), "gemv_ctas_per_sm", "tc_ksplit",
 * "gemm_direct", "gemv_one_kernel" (one-row GEMVs on the grouped kernel, default 1), "l2_prefetch_bytes" (see
 * b200q_set_weight_successor; 0 switches the prefetch off). get also answers "sm_count" and "smem_optin". Options are
 * process-wide tuning and test switches, read by every launch without synchronization: set them once, before the
 * threads that launch are started; the launchers themselves keep no other mutable state. */
int b200q_set_option(const char* name, int value);
int b200q_get_option(const char* name, int* value);

/* The device status word {first failure code, block, detail, failures}: kernels never trap or spin without
 * bound; a wait that gives up records here and the kernel returns. Reading synchronizes the device. */
int b200q_device_status(unsigned int out[4]);
int b200q_reset_device_status(void);
/* First non-zero status a void launcher of part 1 produced since the last call, then cleared. */
int b200q_take_launch_status(void);

/* Diagnostics, in libraries built with -DB200Q_GEMV_TRACE=1 (B200Q_ERR_UNSUPPORTED otherwise: the timestamp sites are
 * left out of the kernels by default). `dev` is device memory for records * 32 uint64; every following GEMV launch takes the next record
 * (wrapping) and its first / last CTA write %globaltimer nanoseconds into slots [0..15] / [16..31]: 0 start,
 * 1 barriers ready, 2 activations staged, 3 first stage landed, 4 done, 5 first weight copy issued, 6 activations
 * quantized, 7 activations in registers, 8 barriers initialised, 9 initial copies issued, 10 activation loads back,
 * 11 first stage consumed, 12 / 13 second stage landed / consumed, 14 / 15 third stage. records = 0 switches it off. */
int b200q_set_trace_buffer(void* dev, int records);

/* One-launch decode GEMV on unquantized activations: x [b_size][stride_x] and dst [b_size][stride_dst] both of
 * element type `elem`; activations are quantized in the kernel's prologue.
 *   act_quant 0: to Q8_1 with the arithmetic of launch_mmvq_gguf_quantize_q8_1_*, so results equal the two-launch
 *                protocol bit for bit (what the reference's CUDA path computes);
 *   act_quant 1: to the reference CPU path's format for the weight type (Q8_K per 256 values for Q4_K / Q6_K,
 *                Q8_0 per 32 for Q8_0), so the integer dot products equal k_quants::matmul's exactly
 *                (crates/inference-tensor/src/quantized/k_quants.rs:2777-2894) and only f32 summation order differs.
 * Host-side counterpart in the reference: fast_mmvq::plain (crates/inference-quant/src/gguf/fast_mmvq.rs:477-665). */
int b200q_gemv(int type, int elem, const void* w, const void* x, void* dst, int K, int N, int stride_x, int stride_dst,
               int b_size, int act_quant, void* stream);

/* Launch order hint, set once when a model is loaded: "the decode launch that follows the one on weight matrix `w`
 * reads `next_w`" (GGUF type next_type, next_N rows of next_K values). Every decode GEMV launch on `w` - through part 1's
 * launch_mmvq_gguf_*_plain symbols as well as b200q_gemv / b200q_gemv_group (keyed by the group's last matrix) - then
 * has each CTA, once its last weight copy is issued, ask L2 (cp.async.bulk.prefetch.L2) for the first
 * "l2_prefetch_bytes" (option; default 64 KB with the "pdl" option on, 256 KB without; -1 restores that default) of
 * the row range the same CTA of the next launch will stream first, so that HBM keeps streaming through the tail of one
 * launch and the gap before the next. A decoder's projections run in
 * a fixed order, so the host registers the chain layer by layer; the hint only moves bytes into L2 early and never
 * changes a result. next_w == NULL forgets `w`; b200q_clear_weight_successors forgets everything (call it before the
 * weights are freed). The table is read-mostly: setting it while other threads launch is safe (a lock), but a launch
 * racing with its own registration may or may not see it. No counterpart in the reference, whose launchers know
 * nothing about the launch after them. */
int b200q_set_weight_successor(const void* w, const void* next_w, int next_type, int next_K, int next_N);
int b200q_clear_weight_successors(void);

/* Grouped decode GEMV: nmat (1..4) weight matrices of GGUF types types[i] with N[i] rows and the same K, applied to the
 * same single activation row x [K] (element type `elem`) in ONE launch; output i goes to dsts[i] [N[i]] in x's type.
 * Activations are quantized to Q8_1 in the prologue, so each output equals b200q_gemv(..., act_quant 0) on that matrix.
 * Takes the place of the reference's fused q/k/v and gate/up matvec launches without their epilogues
 * (launch_mmvq_gguf_<type>_<dst>_fused_qkv / _fused_glu, crates/inference-quant/src/gguf/ffi.rs:1032-1118) and, unlike
 * them, accepts matrices of different types. The pointer arrays are host arrays read during the call. */
int b200q_gemv_group(int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, int elem,
                     const void* x, void* stream);
/* The same with b200q_gemv's act_quant: 1 quantizes the activations to the reference CPU path's format (then the group's
 * matrices must agree on it: all Q8_0, or all K-quants with K a multiple of 256). */
int b200q_gemv_group_act(int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, int elem,
                         const void* x, int act_quant, void* stream);

/* No counterpart in the reference. The decode GEMV for callers that cannot allocate device memory (their memory
 * belongs to a pool of their own, or they may not call cudaMalloc because it synchronizes the device and stalls
 * every other stream): quantizes x [b_size][K] (contiguous rows, element type `elem`) to Q8_1 blocks in a fixed
 * 294,912-byte array inside the library image, then runs the same GEMV as launch_mmvq_gguf_<type>_<elem>_plain on
 * them; dst [b_size][stride_dst] has x's element type and equals that two-launch pair's output. Limits: b_size <= 8
 * and K padded to 512 <= 32768, else B200Q_ERR_TOO_LARGE. Allocates and frees nothing. The first call on a device
 * looks the array's address up (cudaGetSymbolAddress) and should therefore come before any stream capture. All
 * calls on a device share the one array: nothing in it needs clearing between calls (each call rewrites every block
 * it later reads, padding included), but two calls whose kernels can overlap on the GPU - different streams without
 * an ordering between them - race on it. Every GPU that loads the library holds the array until the process exits. */
int b200q_gemv_static_scratch(int type, int elem, const void* w, const void* x, void* dst, int K, int N, int stride_dst,
                              int b_size, void* stream);

/* Prefill GEMM on the tcgen05 tensor cores: y[M][ldy] = x[M][ldx] . W[N][K]^T with x, y of element type `elem`
 * (B200Q_BF16 or B200Q_F16), f32 accumulation in tensor memory. Weights are dequantized tile by tile inside the
 * kernel; activations are not quantized. Needs K a multiple of 64, x 16-byte aligned with ldx * 2 a multiple of 16.
 * Host-side counterpart in the reference: fast_mmq::plain (crates/inference-quant/src/gguf/fast_mmq.rs:604-715,842-845),
 * which quantizes activations to Q8_1 blocks and runs launch_mmq_gguf_<type> (ffi.rs:911-927). */
int b200q_gemm(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, void* stream);

/* Small batches (M = 1..16 activation rows, B200Q_ERR_TOO_LARGE above) on the tcgen05 tensor cores with 8-bit integer
 * operands: y[M][ldy] = x[M][ldx] . W[N][K]^T, x and y of element type `elem` (f32, f16 or bf16). Two launches on
 * `stream`: x is quantized into `workspace` (int8, one f16-rounded scale d = amax / 127 and the integer sum per 32
 * values: the layout kernel mmvq_tc_quantize of the reference, mmvq_gguf/mmvq_quantize.cu:157-190, computes the same
 * values), then one persistent CTA per SM streams its share of the packed weight rows once, unpacks them to int8 and
 * multiplies 128 rows x 32 k blocks by all rows of x with tcgen05.mma kind::i8; block scales are applied in f32.
 * Takes the place of the reference's tensor-core matvec tier for 2..16 rows: fast_mmvq::tiled_plain
 * (crates/inference-quant/src/gguf/fast_mmvq.rs:2049-2126) with launch_mmvq_tc_quantize_<elem> +
 * launch_mmvq_tc_gguf_<type>_<elem>_plain (ffi.rs:631-652,954-998; kernel mmvq_gguf/mmvq_tc_k.cuh:221-329).
 * Needs K a multiple of 256, w 16-byte aligned with a row size that is a multiple of 16 bytes (Q6_K: K a multiple of
 * 2048), workspace 128-byte aligned and at least b200q_gemv_tc_workspace_bytes(type, K) bytes (0 = unsupported K;
 * 18 K bytes, 34 K for Q6_K, plus 1.3 MB for the partial outputs of matrices that are split along K);
 * the workspace is the caller's, as the reference's activation scratch is (gguf/thread_workspace.rs:94-146), and
 * must not be shared by calls that can overlap on the GPU. */
long long b200q_gemv_tc_workspace_bytes(int type, int K);
int b200q_gemv_tc(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, void* workspace,
                  long long workspace_bytes, void* stream);

/* One-shot sum all-reduce of a small vector over NVLink peer memory, for the partial outputs of row-parallel matmuls
 * at decode (the exchange the reference does with an NCCL all-reduce in SumAllReduce,
 * crates/inference-quant/src/distributed/mod.rs:516-670; distributed/layers.rs:814-1190). Every rank calls it with the
 * same n and elem; out = sum over ranks of in, added in rank order in f32, so all ranks hold identical bits; in == out
 * is allowed. `bufs` is a host array of `world` device pointers: every rank's exchange buffer as mapped in THIS
 * process (bufs[rank] is the local one), each b200q_peer_allreduce_buffer_bytes(capacity) bytes (1 KB + 64 capacity: per
 * path - this function, b200q_gemv_allreduce - and call parity an inbox per source rank of twice the vector's size,
 * because every 8 bytes travel together with the number of the call they belong to), zeroed once before the first call
 * and otherwise touched only by these two functions; capacity (bytes, multiple of 16) bounds n * sizeof(elem).
 * Needs 16-byte aligned in / out and n * sizeof(elem) a multiple of 16; world <= 8. Device-side sequence numbers only:
 * captured calls can be replayed. A rank that never arrives makes the others give up after about a second, set the
 * device status word (b200q_device_status) and leave `out` unwritten. */
long long b200q_peer_allreduce_buffer_bytes(long long capacity);
int b200q_peer_allreduce(const void* const* bufs, int rank, int world, long long capacity, int elem, const void* in, void* out,
                         long long n, void* stream);

/* The row-parallel matmul and its exchange in ONE launch (the reference runs them as two operations:
 * RowParallelLayer::forward_raw, crates/inference-quant/src/distributed/layers.rs:1036-1046): b200q_gemv on contiguous
 * x [b_size][K] -> dst [b_size][N] in which every CTA, when its rows are done, sends them to all ranks and adds up what
 * the same CTA of every rank sent (b200q_peer_allreduce's protocol, piece by piece), so that after the launch every
 * rank's dst holds the sum of all ranks' partial outputs, bit-identical on all ranks and to b200q_gemv followed by
 * b200q_peer_allreduce. Same `bufs`, `capacity` and calling discipline as b200q_peer_allreduce (all ranks, same order);
 * N * sizeof(elem) must be a multiple of 8, b_size * N * sizeof(elem) at most `capacity`, dst 8-byte aligned and
 * contiguous; B200Q_ERR_UNSUPPORTED otherwise or where b200q_gemv has
 * no staged kernel for the shape (then: the two separate calls). world == 1 is a plain b200q_gemv. */
int b200q_gemv_allreduce(int type, int elem, const void* w, const void* x, void* dst, int K, int N, int b_size,
                         const void* const* bufs, int rank, int world, long long capacity, void* stream);

/* Weight quantizers on the device: n f32 values at x (device memory; n a multiple of the type's block: 32 for Q8_0,
 * 256 otherwise) -> packed blocks at out, byte for byte what the reference's CPU quantizer writes in its default mode
 * without an importance matrix (QTensor::quantize, crates/inference-tensor/src/quantized/mod.rs:903-918; Q8_0
 * quantized/mod.rs:43-56, Q4_K k_quants.rs:1949-2015 with utils.rs:268-361, Q6_K k_quants.rs:2590-2646 with
 * utils.rs:135-264). The reference has device quantizers for Q6_K and Q8_0 only
 * (crates/inference-quant/kernels/cuda/gguf_quantize/k_quantize_instance_ggufq.cu:203-242) and runs Q4_K on the host. */
int b200q_quantize(int type, const void* x, void* out, long long n, void* stream);

/* Packed rows back to values of element type `elem`: b200q_dequantize all nrows rows of K values (to_float,
 * k_quants.rs:905-921,2096-2123,2649-2680); b200q_get_rows the rows ids[0..n_ids) of a table of nrows_w rows (the
 * quantized embedding gather, crates/inference-tensor/src/quantized/cuda.rs:151-242; ids are device int32). An id
 * outside the table gives a row of zeros and code 6 in the device status word. */
int b200q_dequantize(int type, int elem, const void* w, void* out, long long nrows, int K, void* stream);
int b200q_get_rows(int type, int elem, const void* w, const int32_t* ids, void* out, long long n_ids, int K, long long nrows_w,
                   void* stream);

/* out = {staged kernel?, grid, dynamic smem bytes, stages, rows per stage, warps per row, stage bytes, rows per unit of
 *        the CTAs' row partition (the 16-byte alignment unit, or a whole stage for short launches), item slots per lane,
 *        register-resident slots} */
int b200q_gemv_plan(int type, int K, int N, int b_size, int out[10]);

#ifdef __cplusplus
}
#endif
#endif /* INFERENCEQUANT_B200_H */

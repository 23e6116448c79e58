// The status-returning half of the C ABI (include/inferencequant_b200.h): options, status words, and the
// one-launch GEMV that quantizes activations in its prologue.
#include <cstdio>
#include <cstring>

#include "common.cuh"
#include "peer_allreduce.cuh"
#include "runtime.h"

#ifndef B200Q_GEMV_TRACE
#define B200Q_GEMV_TRACE 0
#endif

namespace b200q {
int gemv_q4_k(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
int gemv_q6_k(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
int gemv_q8_0(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
void gemv_describe(int type, int K, int N, int b, int* out);
int gemv_group(int elem, int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, const void* x,
               cudaStream_t s, const PeerExchange* px, int act_mode);
int gemm_dispatch(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, cudaStream_t s);
int gemv_tc_dispatch(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, void* workspace, cudaStream_t s);
size_t gemv_tc_workspace_bytes(int type, int K);
long long peer_allreduce_buffer_bytes(long long capacity);
int quantize_weights(int type, const float* x, void* out, long long n, cudaStream_t s);
int dequantize_rows(int type, int elem, const void* w, const int* ids, void* out, long long nrows_out, int K, long long nrows_w,
                    cudaStream_t s);
int fill_peer_exchange(PeerExchange& px, const void* const* bufs, int rank, int world, long long capacity);
int peer_allreduce(const void* const* bufs, int rank, int world, long long capacity, int elem, const void* in, void* out, long long n,
                   cudaStream_t s);

static thread_local char t_error[320] = "";
int set_error(int code, const char* msg) {
    std::snprintf(t_error, sizeof t_error, "%s", msg);
    return code;
}
}  // namespace b200q

using namespace b200q;

extern "C" {

// Checked by the reference's loader against the id compiled into the host
// (crates/inference-tensor/src/kernel_library.rs:288-297). A host built for this library bakes the same string.
extern const char inference_kernel_build_id[] = "b200q-sm100a-0.1";

const char* b200q_version(void) { return "0.1.0"; }
const char* b200q_last_error(void) { return t_error; }

int b200q_set_option(const char* name, int value) {
    RuntimeInfo& rt = runtime_info_mut();
    if (!std::strcmp(name, "pdl")) rt.use_pdl = value;
    else if (!std::strcmp(name, "force_simple_gemv")) rt.force_simple = value;
    else if (!std::strcmp(name, "gemv_stage_bytes")) {
        if (value < 1024) return set_error(B200Q_ERR_INVALID, "gemv_stage_bytes must be >= 1024");
        rt.gemv_stage_target = value;
    } else if (!std::strcmp(name, "tc_ksplit")) {
        rt.tc_ksplit = value ? 1 : 0;
    } else if (!std::strcmp(name, "gemm_direct")) {
        rt.gemm_direct = value ? 1 : 0;
    } else if (!std::strcmp(name, "l2_prefetch_bytes")) {
        if (value < -1) return set_error(B200Q_ERR_INVALID, "l2_prefetch_bytes must be >= 0, or -1 for the default of the launch mode");
        rt.l2_prefetch_bytes = value < 0 ? -1 : (value & ~15);
    } else if (!std::strcmp(name, "gemv_one_kernel")) {
        rt.gemv_one_kernel = value ? 1 : 0;
    } else if (!std::strcmp(name, "gemv_passes")) {
        if (value < 0 || value > 2) return set_error(B200Q_ERR_INVALID, "gemv_passes is 0 (planner's choice), 1 or 2");
        rt.gemv_passes = value;
    } else if (!std::strcmp(name, "gemv_pass_limit_bytes")) {
        if (value < 1024) return set_error(B200Q_ERR_INVALID, "gemv_pass_limit_bytes must be >= 1024");
        rt.gemv_pass_limit = value;
    } else if (!std::strcmp(name, "gemv_ctas_per_sm")) {
        if (value != 1 && value != 2) return set_error(B200Q_ERR_INVALID, "gemv_ctas_per_sm is 1 or 2");
        rt.gemv_ctas_per_sm = value;
    } else {
        return set_error(B200Q_ERR_INVALID, "unknown option");
    }
    return B200Q_OK;
}

int b200q_get_option(const char* name, int* value) {
    const RuntimeInfo& rt = runtime_info();
    if (!std::strcmp(name, "pdl")) *value = rt.use_pdl;
    else if (!std::strcmp(name, "force_simple_gemv")) *value = rt.force_simple;
    else if (!std::strcmp(name, "gemv_stage_bytes")) *value = rt.gemv_stage_target;
    else if (!std::strcmp(name, "gemv_ctas_per_sm")) *value = rt.gemv_ctas_per_sm;
    else if (!std::strcmp(name, "gemv_one_kernel")) *value = rt.gemv_one_kernel;
    else if (!std::strcmp(name, "gemv_passes")) *value = rt.gemv_passes;
    else if (!std::strcmp(name, "gemv_pass_limit_bytes")) *value = rt.gemv_pass_limit;
    else if (!std::strcmp(name, "gemm_direct")) *value = rt.gemm_direct;
    else if (!std::strcmp(name, "tc_ksplit")) *value = rt.tc_ksplit;
    else if (!std::strcmp(name, "l2_prefetch_bytes")) *value = l2_prefetch_bytes_effective(rt);
    else if (!std::strcmp(name, "sm_count")) *value = rt.sm_count;
    else if (!std::strcmp(name, "smem_optin")) *value = rt.smem_optin;
    else return set_error(B200Q_ERR_INVALID, "unknown option");
    return B200Q_OK;
}

// Copies the device status word {code, block, detail, count} of the current device to `out` (synchronizes the device).
int b200q_device_status(unsigned int out[4]) {
    unsigned int* p = status_ptr();
    if (!p) return set_error(B200Q_ERR_INVALID, "no CUDA device");
    cudaError_t e = cudaMemcpy(out, p, 4 * sizeof(unsigned int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return set_error((int)e, cudaGetErrorString(e));
    return B200Q_OK;
}

int b200q_reset_device_status(void) {
    unsigned int* p = status_ptr();
    if (!p) return set_error(B200Q_ERR_INVALID, "no CUDA device");
    cudaError_t e = cudaMemset(p, 0, 4 * sizeof(unsigned int));
    if (e != cudaSuccess) return set_error((int)e, cudaGetErrorString(e));
    return B200Q_OK;
}

// Diagnostics: `dev` points at records * 32 u64; every following GEMV launch takes the next record and its first / last CTA
// write nanosecond timestamps into slots [0..15] / [16..31] (slot meanings: include/inferencequant_b200.h). records = 0: off.
int b200q_set_trace_buffer(void* dev, int records) {
#if B200Q_GEMV_TRACE
    set_trace_buffer(static_cast<unsigned long long*>(dev), dev ? records : 0);
    return B200Q_OK;
#else
    if (dev != nullptr && records > 0) return set_error(B200Q_ERR_UNSUPPORTED, "this library was built without -DB200Q_GEMV_TRACE=1");
    return B200Q_OK;
#endif
}

// First non-zero status a void launcher produced since the last call (then cleared).
int b200q_take_launch_status(void) { return take_launch_status(); }

static int gemv_one_launch(int type, int elem, const void* w, const void* x, void* dst, int K, int N, int stride_x, int stride_dst,
                           int b_size, int act_quant, const PeerExchange* px, void* stream) {
    if (act_quant != 0 && act_quant != 1) return set_error(B200Q_ERR_INVALID, "act_quant is 0 (Q8_1) or 1 (CPU path's format)");
    const int mode = act_quant == 0 ? 1 : 2;  // ACT_RAW_Q8_1 / ACT_RAW_CPU
    if (!w || !x || !dst) return set_error(B200Q_ERR_INVALID, "null pointer");
    if (b_size < 1 || b_size > 8) return set_error(B200Q_ERR_UNSUPPORTED, "b200q_gemv takes 1..8 activation rows");
    if (K <= 0 || K % type_block_elems(type) != 0) return set_error(B200Q_ERR_INVALID, "K is not a multiple of the block size");
    int rc;
    cudaStream_t s = (cudaStream_t)stream;
    if (type == TYPE_Q4_K) rc = gemv_q4_k(elem, w, x, dst, K, N, stride_x, stride_dst, b_size, mode, px, s);
    else if (type == TYPE_Q6_K) rc = gemv_q6_k(elem, w, x, dst, K, N, stride_x, stride_dst, b_size, mode, px, s);
    else if (type == TYPE_Q8_0) rc = gemv_q8_0(elem, w, x, dst, K, N, stride_x, stride_dst, b_size, mode, px, s);
    else return set_error(B200Q_ERR_UNSUPPORTED, "weight type is not Q8_0, Q4_K or Q6_K");
    take_launch_status();
    if (rc == B200Q_ERR_UNSUPPORTED)
        return set_error(rc, "no one-launch GEMV for this shape or alignment: quantize to Q8_1 and use launch_mmvq_gguf_*_plain");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "gemv failed");
    return B200Q_OK;
}

int b200q_gemv(int type, int elem, const void* w, const void* x, void* dst, int K, int N, int stride_x, int stride_dst,
               int b_size, int act_quant, void* stream) {
    return gemv_one_launch(type, elem, w, x, dst, K, N, stride_x, stride_dst, b_size, act_quant, nullptr, stream);
}

// "The launch after the one on `w` reads `next_w`" (a matrix of GGUF type next_type with next_N rows of next_K values);
// next_w == NULL forgets w. Read by every decode GEMV launch on w from then on.
int b200q_set_weight_successor(const void* w, const void* next_w, int next_type, int next_K, int next_N) {
    if (!w) return set_error(B200Q_ERR_INVALID, "null pointer");
    if (next_w == nullptr) {
        set_weight_successor(w, nullptr);
        return B200Q_OK;
    }
    if (type_block_bytes(next_type) == 0 || next_K <= 0 || next_N <= 0 || next_K % type_block_elems(next_type) != 0)
        return set_error(B200Q_ERR_INVALID, "b200q_set_weight_successor: bad type or shape of the successor");
    const WeightSuccessor succ{next_w, next_type, next_K, next_N};
    set_weight_successor(w, &succ);
    return B200Q_OK;
}

int b200q_clear_weight_successors(void) {
    clear_weight_successors();
    return B200Q_OK;
}

// Grouped decode GEMV: nmat (1..4) weight matrices with the same K applied to the same activation row x [K] in one launch.
static int gemv_group_checked(int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, int elem,
                              const void* x, int act_quant, void* stream) {
    if (!types || !ws || !dsts || !Ns || !x) return set_error(B200Q_ERR_INVALID, "null pointer");
    if (nmat < 1 || nmat > 4) return set_error(B200Q_ERR_INVALID, "b200q_gemv_group takes 1..4 matrices");
    if (act_quant != 0 && act_quant != 1) return set_error(B200Q_ERR_INVALID, "act_quant is 0 (Q8_1) or 1 (CPU path's format)");
    const int rc = gemv_group(elem, nmat, types, ws, dsts, Ns, K, x, (cudaStream_t)stream, nullptr, act_quant == 0 ? 1 : 2);
    if (rc == B200Q_ERR_UNSUPPORTED)
        return set_error(rc, "group not supported (K must be a multiple of 128 - 256 for K-quants with act_quant 1 -, weights 16-byte "
                             "aligned, and with act_quant 1 all matrices Q8_0 or none): launch the matrices one by one");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "grouped gemv failed");
    return B200Q_OK;
}
int b200q_gemv_group(int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, int elem,
                     const void* x, void* stream) {
    return gemv_group_checked(nmat, types, ws, dsts, Ns, K, elem, x, 0, stream);
}
// The same with the activation format chosen as in b200q_gemv (act_quant 1: the reference CPU path's Q8_K / Q8_0).
int b200q_gemv_group_act(int nmat, const int* types, const void* const* ws, void* const* dsts, const int* Ns, int K, int elem,
                         const void* x, int act_quant, void* stream) {
    return gemv_group_checked(nmat, types, ws, dsts, Ns, K, elem, x, act_quant, stream);
}

// Prefill GEMM on the tensor cores: y[M][ldy] = x[M][ldx] . W[N][K]^T, x and y of element type `elem` (bf16 or f16).
int b200q_gemm(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, void* stream) {
    if (!w || !x || !y) return set_error(B200Q_ERR_INVALID, "null pointer");
    if (type_block_bytes(type) == 0) return set_error(B200Q_ERR_UNSUPPORTED, "weight type is not Q8_0, Q4_K or Q6_K");
    if (elem != ELEM_BF16 && elem != ELEM_F16) return set_error(B200Q_ERR_UNSUPPORTED, "b200q_gemm takes bf16 or f16 activations");
    const int rc = gemm_dispatch(type, elem, w, x, y, M, N, K, ldx, ldy, (cudaStream_t)stream);
    if (rc == B200Q_ERR_UNSUPPORTED)
        return set_error(rc, "b200q_gemm needs K a multiple of 64 and of the weight type's block size, x 16-byte aligned with ldx * 2 a "
                             "multiple of 16, weights 2-byte aligned (Q4_K: 16-byte), and a driver that provides cuTensorMapEncodeTiled");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "gemm failed");
    return B200Q_OK;
}

// Small batches (1..16 rows) on the tensor cores with int8 operands: quantizes x into `workspace`, then streams the weights once.
long long b200q_gemv_tc_workspace_bytes(int type, int K) {
    if (type_block_bytes(type) == 0 || K <= 0 || K % 256 != 0) return 0;
    return (long long)gemv_tc_workspace_bytes(type, K);
}

int b200q_gemv_tc(int type, int elem, const void* w, const void* x, void* y, int M, int N, int K, int ldx, int ldy, void* workspace,
                  long long workspace_bytes, void* stream) {
    if (!w || !x || !y || !workspace) return set_error(B200Q_ERR_INVALID, "null pointer");
    if (type_block_bytes(type) == 0) return set_error(B200Q_ERR_UNSUPPORTED, "weight type is not Q8_0, Q4_K or Q6_K");
    if (elem != ELEM_BF16 && elem != ELEM_F16 && elem != ELEM_F32) return set_error(B200Q_ERR_INVALID, "unknown element type");
    if (M > 16) return set_error(B200Q_ERR_TOO_LARGE, "b200q_gemv_tc takes at most 16 activation rows");
    if (K <= 0 || K % 256 != 0) return set_error(B200Q_ERR_UNSUPPORTED, "b200q_gemv_tc needs K a multiple of 256");
    if (workspace_bytes < (long long)gemv_tc_workspace_bytes(type, K)) return set_error(B200Q_ERR_INVALID, "workspace smaller than b200q_gemv_tc_workspace_bytes");
    const int rc = gemv_tc_dispatch(type, elem, w, x, y, M, N, K, ldx, ldy, workspace, (cudaStream_t)stream);
    if (rc == B200Q_ERR_UNSUPPORTED)
        return set_error(rc, "b200q_gemv_tc needs 16-byte aligned weights whose rows are a multiple of 16 bytes (Q6_K: K a multiple of 2048)");
    if (rc == B200Q_ERR_INVALID) return set_error(rc, "workspace must be 128-byte aligned");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "gemv_tc failed");
    return B200Q_OK;
}

// One-shot sum all-reduce over peer-mapped buffers (tensor-parallel decode): see peer_allreduce.cu.
long long b200q_peer_allreduce_buffer_bytes(long long capacity) {
    if (capacity <= 0 || capacity % 16 != 0) return 0;
    return peer_allreduce_buffer_bytes(capacity);
}

int b200q_peer_allreduce(const void* const* bufs, int rank, int world, long long capacity, int elem, const void* in, void* out,
                         long long n, void* stream) {
    if (!bufs || !in || !out) return set_error(B200Q_ERR_INVALID, "null pointer");
    if (elem != ELEM_BF16 && elem != ELEM_F16 && elem != ELEM_F32) return set_error(B200Q_ERR_INVALID, "unknown element type");
    const int rc = peer_allreduce(bufs, rank, world, capacity, elem, in, out, n, (cudaStream_t)stream);
    if (rc == B200Q_ERR_INVALID) return set_error(rc, "b200q_peer_allreduce: 1..8 ranks, 16-byte aligned buffers, capacity a multiple of 16");
    if (rc == B200Q_ERR_TOO_LARGE) return set_error(rc, "b200q_peer_allreduce: the vector is larger than the staging capacity");
    if (rc == B200Q_ERR_UNSUPPORTED) return set_error(rc, "b200q_peer_allreduce needs 16-byte aligned in / out and a size that is a multiple of 16 bytes");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "peer all-reduce failed");
    return B200Q_OK;
}

// Row-parallel matmul and its sum over the ranks in ONE launch: b200q_gemv in which every CTA exchanges its own rows of the
// output with the same CTA of the other ranks (peer_allreduce.cuh) and stores their sum.
int b200q_gemv_allreduce(int type, int elem, const void* w, const void* x, void* dst, int K, int N, int b_size, const void* const* bufs,
                         int rank, int world, long long capacity, void* stream) {
    if (!bufs) return set_error(B200Q_ERR_INVALID, "null pointer");
    PeerExchange px{};
    if (fill_peer_exchange(px, bufs, rank, world, capacity) != 0)
        return set_error(B200Q_ERR_INVALID, "b200q_gemv_allreduce: 1..8 ranks, 16-byte aligned buffers, capacity a multiple of 16");
    return gemv_one_launch(type, elem, w, x, dst, K, N, K, N, b_size, 0, world > 1 ? &px : nullptr, stream);
}

// f32 values on the device -> packed blocks, byte for byte the reference CPU quantizer's (default mode).
int b200q_quantize(int type, const void* x, void* out, long long n, void* stream) {
    if (!x || !out) return set_error(B200Q_ERR_INVALID, "null pointer");
    const int rc = quantize_weights(type, static_cast<const float*>(x), out, n, (cudaStream_t)stream);
    if (rc == B200Q_ERR_UNSUPPORTED) return set_error(rc, "weight type is not Q8_0, Q4_K or Q6_K");
    if (rc == B200Q_ERR_INVALID) return set_error(rc, "the number of values is not a multiple of the block size, or the output is not 2-byte aligned");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "quantize failed");
    return B200Q_OK;
}

// Packed rows -> values of element type `elem`: all rows (to_float), or the rows `ids` names (embedding gather).
int b200q_dequantize(int type, int elem, const void* w, void* out, long long nrows, int K, void* stream) {
    if (!w || !out) return set_error(B200Q_ERR_INVALID, "null pointer");
    const int rc = dequantize_rows(type, elem, w, nullptr, out, nrows, K, nrows, (cudaStream_t)stream);
    if (rc == B200Q_ERR_UNSUPPORTED) return set_error(rc, "weight type is not Q8_0, Q4_K or Q6_K");
    if (rc == B200Q_ERR_INVALID) return set_error(rc, "b200q_dequantize: K must be a multiple of the block size, elem f32 / f16 / bf16");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "dequantize failed");
    return B200Q_OK;
}

int b200q_get_rows(int type, int elem, const void* w, const int32_t* ids, void* out, long long n_ids, int K, long long nrows_w, void* stream) {
    if (!w || !out || !ids) return set_error(B200Q_ERR_INVALID, "null pointer");
    const int rc = dequantize_rows(type, elem, w, ids, out, n_ids, K, nrows_w, (cudaStream_t)stream);
    if (rc == B200Q_ERR_UNSUPPORTED) return set_error(rc, "weight type is not Q8_0, Q4_K or Q6_K");
    if (rc == B200Q_ERR_INVALID) return set_error(rc, "b200q_get_rows: K must be a multiple of the block size, elem f32 / f16 / bf16");
    if (rc != 0) return set_error(rc, rc > 0 ? cudaGetErrorString((cudaError_t)rc) : "get_rows failed");
    return B200Q_OK;
}

// out[10] = {staged, grid, smem bytes, stages, rows per stage, warps per row, stage bytes, row alignment,
//            item slots per lane, register-resident slots}
int b200q_gemv_plan(int type, int K, int N, int b_size, int out[10]) {
    if (type_block_bytes(type) == 0 || K <= 0 || K % type_block_elems(type) != 0 || b_size < 1 || b_size > 8)
        return set_error(B200Q_ERR_INVALID, "bad shape");
    gemv_describe(type, K, N, b_size, out);
    return B200Q_OK;
}

}  // extern "C"

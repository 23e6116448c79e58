// The reference's fused decode matvecs (crates/inference-quant/kernels/cuda/mmvq_gguf/mmvq_gguf.cuh:761-962, symbols
// crates/inference-quant/src/gguf/ffi.rs:1032-1118), on Q8_1 activation blocks as its host passes them:
//
//  * fused_glu: out[j][row] = act(gate[row] . y[j]) * (up[row] . y[j]) - the gate and up projections of an MLP and the
//    gated activation in ONE launch. Here: the TMA-ring GEMV with every stage holding the same rows of BOTH matrices, so
//    a warp computes a row's two dot products together (two independent chains: one's latencies hide behind the other)
//    and applies the epilogue in registers. Rounding order as the reference's (mmvq_gguf.cuh:829-836): gate and up are
//    rounded to the output type first, the activation runs in f32 on the rounded gate and is rounded, the product is
//    formed in the output type.
//  * fused_qkv: three matrices of one type on the same activations, each with its own output and row count. One
//    activation row goes through the grouped GEMV (one launch for the three); more rows through three launches of the
//    plain GEMV (same results; the launchers return before any of them has run, as the reference's do).
#include <cmath>

#include "gemv_impl.cuh"

namespace b200q {

// activation ids: crates/inference-quant/kernels/cuda/glu_activation.cuh:4-10 (GluActivationType on the host side)
enum GluActivation : int { GLU_SILU = 0, GLU_GELU = 1, GLU_RELU = 2, GLU_GELU_ERF = 3, GLU_SIGMOID = 4 };

__device__ __forceinline__ float glu_activation(float x, int act) {
    switch (act) {
        case GLU_GELU: {
            const float inner = 0.7978845608f * (x + 0.044715f * (x * x * x));
            return 0.5f * x * (1.0f + tanhf(inner));
        }
        case GLU_RELU: return fmaxf(x, 0.0f);
        case GLU_GELU_ERF: return x * normcdff(x);
        case GLU_SIGMOID: return 1.0f / (1.0f + expf(-x));
        default: return x / (1.0f + expf(-x));  // SiLU, also for unknown ids as in the reference
    }
}

template <typename dst_t> __device__ __forceinline__ dst_t glu_combine(float gate, float up, int act) {
    const dst_t g = from_float<dst_t>(gate), u = from_float<dst_t>(up);
    const dst_t a = from_float<dst_t>(glu_activation(to_float<dst_t>(g), act));
    if constexpr (sizeof(dst_t) == 4) return a * u;
    else return __hmul(a, u);  // one rounding in the output type
}

struct GemvGluParams {
    const uint8_t* wg;   // gate rows, packed
    const uint8_t* wu;   // up rows, packed (same type and shape)
    const void* act;     // Q8_1 blocks [B][stride_act]
    void* dst;           // [B][stride_dst]
    int K, N, stride_act, stride_dst, row_bytes;
    int rows_per_stage;  // rows of EACH matrix a stage holds (a multiple of one pass of all warps)
    int half_bytes;      // offset of the up rows inside a stage (multiple of 16)
    int warps_per_row, items_per_lane, log2_wpr, log2_islots;
    int row_align, units_per_cta, units_extra, nstages, stage_bytes, act_bytes;
    int activation;
    unsigned int* status;
};

// One CTA per SM, 16 consumer warps + 1 producer warp, as gemv_staged_kernel; NREG = register-resident item slots.
template <int TYPE, int B, typename dst_t, int NREG>
__global__ void __launch_bounds__(GEMV_THREADS, 1) gemv_glu_kernel(const GemvGluParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty = full + GEMV_MAX_STAGES;
    uint8_t* acts = smem + GEMV_BARRIER_BYTES;
    const int S = p.nstages, R = p.rows_per_stage, WPR = p.warps_per_row, IPL = p.items_per_lane;
    // cross-warp combine (WPR > 1): per stage and row, WPR partial sums of gate and of up per activation row, and a counter
    float* partial = reinterpret_cast<float*>(acts + p.act_bytes);  // [S][R][WPR][2][B]
    const int partial_floats = WPR > 1 ? S * R * WPR * 2 * B : 0;
    int* counters = reinterpret_cast<int*>(partial + partial_floats);  // [S][R]
    const int counter_ints = WPR > 1 ? S * R : 0;
    uint8_t* ring = acts + p.act_bytes + (((partial_floats + counter_ints) * 4 + 127) & ~127);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_producer = warp == GEMV_CONSUMER_WARPS;
    ActPrefetch<ACT_Q8_1, float> pre;
    if (!is_producer) pre.issue(p.act, B, p.K, p.stride_act, false, tid);

    const int cta = blockIdx.x;
    const int unit0 = cta * p.units_per_cta + min(cta, p.units_extra);
    const int row0 = unit0 * p.row_align;
    int row1 = (unit0 + p.units_per_cta + (cta < p.units_extra ? 1 : 0)) * p.row_align;
    if (row1 > p.N) row1 = p.N;
    if (row1 < row0) row1 = row0;

    if (is_producer && lane == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], GEMV_CONSUMER_WARPS);
        }
        mbar_init_fence();
    }
    for (int i = tid; i < counter_ints; i += GEMV_THREADS) counters[i] = 0;
    __syncthreads();

    if (is_producer) {
        if (lane == 0) {
            bool ok = true;
            int s = 0, g = 0;
            uint32_t ph = 1;
            for (int r = row0; r < row1 && ok; r += R, ++g) {
                if (g >= S) {
                    ok = mbar_wait_bounded(&empty[s], ph);
                    if (!ok) { record_failure(p.status, STATUS_WAIT_EMPTY_TIMEOUT, g); break; }
                }
                const int rows = min(R, row1 - r);
                const uint32_t bytes = ((uint32_t)rows * (uint32_t)p.row_bytes + 15u) & ~15u;
                uint8_t* st = ring + (size_t)s * p.stage_bytes;
                mbar_arrive_expect_tx(&full[s], 2 * bytes);
                bulk_copy_g2s(st, p.wg + (size_t)r * p.row_bytes, bytes, &full[s]);
                bulk_copy_g2s(st + p.half_bytes, p.wu + (size_t)r * p.row_bytes, bytes, &full[s]);
                if (++s == S) {
                    s = 0;
                    ph ^= 1u;
                }
            }
            if (!ok) {  // let the copies already issued land before the CTA may exit
                for (int q = max(0, g - S); q < g; ++q)
                    if (!mbar_wait_bounded(&full[q % S], (q / S) & 1)) {
                        record_failure(p.status, STATUS_WAIT_DRAIN_TIMEOUT, q);
                        break;
                    }
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    stage_acts_q8_1<B>(acts, reinterpret_cast<const uint8_t*>(p.act), p.K, p.stride_act, tid, GEMV_CONSUMER_THREADS, pre);
    named_bar_sync(1, GEMV_CONSUMER_THREADS);

    const int nrec = p.K / 64;
    const int items = p.K / 128;
    const int islots = 1 << p.log2_islots;
    const int rpw = 32 >> p.log2_islots;
    const int lane_i = lane & (islots - 1), lane_r = lane >> p.log2_islots;
    const int nrg = GEMV_CONSUMER_WARPS >> p.log2_wpr;
    const int wgroup = warp >> p.log2_wpr, wslice = warp & (WPR - 1);
    const int row_slot = wgroup * rpw + lane_r;
    const int rows_per_pass = nrg * rpw;
    const int item0 = wslice * 32 + lane_i;
    const int item_step = 32 * WPR;
    const uint32_t acts_addr = smem_u32(acts);
    const uint32_t ring_addr = smem_u32(ring);
    const uint32_t act_row_bytes = (uint32_t)nrec * ACT_REC_BYTES;
    dst_t* dst = reinterpret_cast<dst_t*>(p.dst);

    Acts<TYPE> areg[NREG > 0 ? B : 1][NREG > 0 ? NREG : 1];
    if (NREG > 0) {
#pragma unroll
        for (int b = 0; b < B; ++b)
#pragma unroll
            for (int j = 0; j < (NREG > 0 ? NREG : 1); ++j)
                if (item0 + j * item_step < items) areg[b][j].load(acts_addr + b * act_row_bytes, item0 + j * item_step);
    }

    bool alive = true;
    int s = 0;
    uint32_t ph = 0;
    int rot = 0, rot_step = R;
    while (rot_step >= rows_per_pass) rot_step -= rows_per_pass;
    for (int it = 0, rbase = row0; rbase < row1; ++it, rbase += R) {
        if (alive && !mbar_wait_bounded(&full[s], ph)) {
            record_failure(p.status, STATUS_WAIT_FULL_TIMEOUT, it);
            alive = false;
        }
        const uint32_t st = ring_addr + (uint32_t)s * (uint32_t)p.stage_bytes;
        const int rows_here = min(R, row1 - rbase);
        const int my_slot = row_slot >= rot ? row_slot - rot : row_slot - rot + rows_per_pass;
        for (int pass0 = 0; pass0 < rows_here; pass0 += rows_per_pass) {  // warp-uniform trip count
            const int r_in = pass0 + my_slot;
            const bool has_row = r_in < rows_here;
            float acc[2][B];  // [gate, up]
#pragma unroll
            for (int u = 0; u < 2; ++u)
#pragma unroll
                for (int b = 0; b < B; ++b) acc[u][b] = 0.0f;
            const uint32_t row_addr = st + (uint32_t)(has_row ? r_in : 0) * (uint32_t)p.row_bytes;
            if constexpr (NREG > 0) {
                // unconditional on clamped addresses, masked afterwards: one basic block, two independent chains
#pragma unroll
                for (int j = 0; j < NREG; ++j) {
                    const int item = item0 + j * item_step;
                    const bool item_ok = item < items;
                    Weights<TYPE> W[2];
                    W[0].load(row_addr, item_ok ? item : 0);
                    W[1].load(row_addr + (uint32_t)p.half_bytes, item_ok ? item : 0);
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int b = 0; b < B; ++b) {
                            const float d = dot(W[u], areg[b][j]);
                            acc[u][b] += (alive && has_row && item_ok) ? d : 0.0f;
                        }
                }
            } else if (alive && has_row) {
                for (int j = 0; j < IPL; ++j) {
                    const int item = item0 + j * item_step;
                    if (item < items) {
                        Weights<TYPE> W[2];
                        W[0].load(row_addr, item);
                        W[1].load(row_addr + (uint32_t)p.half_bytes, item);
#pragma unroll
                        for (int b = 0; b < B; ++b) {
                            Acts<TYPE> A;
                            A.load(acts_addr + b * act_row_bytes, item);
                            acc[0][b] += dot(W[0], A);
                            acc[1][b] += dot(W[1], A);
                        }
                    }
                }
            }
#pragma unroll
            for (int m = 16; m > 0; m >>= 1) {
                if (m < islots) {
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int b = 0; b < B; ++b) acc[u][b] += __shfl_xor_sync(0xffffffffu, acc[u][b], m);
                }
            }
            if (lane_i == 0 && has_row) {
                if (WPR == 1) {
#pragma unroll
                    for (int b = 0; b < B; ++b)
                        dst[(size_t)b * p.stride_dst + rbase + r_in] = glu_combine<dst_t>(acc[0][b], acc[1][b], p.activation);
                } else {
                    // the last of the WPR warps to arrive adds the partial sums in slice order and writes the row
                    float* part = partial + ((size_t)(s * R + r_in) * WPR) * 2 * B;
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int b = 0; b < B; ++b) part[(wslice * 2 + u) * B + b] = acc[u][b];
                    __threadfence_block();
                    const int arrived = atomicAdd(&counters[s * R + r_in], 1);
                    if (arrived == WPR - 1) {
                        __threadfence_block();
                        counters[s * R + r_in] = 0;
#pragma unroll
                        for (int b = 0; b < B; ++b) {
                            float g = 0.0f, u = 0.0f;
                            for (int w = 0; w < WPR; ++w) {
                                g += reinterpret_cast<volatile float*>(part)[(w * 2 + 0) * B + b];
                                u += reinterpret_cast<volatile float*>(part)[(w * 2 + 1) * B + b];
                            }
                            dst[(size_t)b * p.stride_dst + rbase + r_in] = glu_combine<dst_t>(g, u, p.activation);
                        }
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[s]);
        if (++s == S) {
            s = 0;
            ph ^= 1u;
        }
        rot += rot_step;
        if (rot >= rows_per_pass) rot -= rows_per_pass;
    }
}

// Shapes the ring kernel does not take (K not a multiple of 128, unaligned weights, no ring that fits): a warp per row,
// byte-granular loads, both dot products per 32-value group.
template <int TYPE, int B, typename dst_t>
__global__ void __launch_bounds__(256) gemv_glu_simple_kernel(const uint8_t* __restrict__ wg, const uint8_t* __restrict__ wu,
                                                              const uint8_t* __restrict__ vy, dst_t* __restrict__ dst, int K, int N,
                                                              int stride_act, int stride_dst, int activation) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= N) return;
    const size_t row_bytes = (size_t)(K / type_block_elems(TYPE)) * type_block_bytes(TYPE);
    float acc[2][B];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int b = 0; b < B; ++b) acc[u][b] = 0.0f;
    for (int kb = lane; kb < K / 32; kb += 32) {
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const uint8_t* rp = (u == 0 ? wg : wu) + (size_t)row * row_bytes;
            int wq[32];
            float s0 = 0.0f, s1 = 0.0f, mn = 0.0f;
            if (TYPE == TYPE_Q8_0) {
                const uint8_t* blk = rp + (size_t)kb * Q8_0_BYTES;
                s0 = half_bits_to_float((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
                for (int l = 0; l < 32; ++l) wq[l] = ld_i8(blk + 2 + l);
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
                s0 = d * (float)ld_i8(sb + 192 + 8 * n + 2 * qd);
                s1 = d * (float)ld_i8(sb + 192 + 8 * n + 2 * qd + 1);
            }
#pragma unroll
            for (int b = 0; b < B; ++b) {
                const uint8_t* ab = vy + ((size_t)b * stride_act + kb) * Q8_1_BYTES;
                const float d8 = half_bits_to_float((uint32_t)ab[0] | ((uint32_t)ab[1] << 8));
                int d0 = 0, d1 = 0, s8 = 0;
                for (int l = 0; l < 16; ++l) { const int a = ld_i8(ab + 4 + l); d0 += wq[l] * a; s8 += a; }
                for (int l = 16; l < 32; ++l) { const int a = ld_i8(ab + 4 + l); d1 += wq[l] * a; s8 += a; }
                if (TYPE == TYPE_Q6_K) acc[u][b] += d8 * (s0 * (float)d0 + s1 * (float)d1);
                else if (TYPE == TYPE_Q4_K) acc[u][b] += s0 * d8 * (float)(d0 + d1) - mn * d8 * (float)s8;
                else acc[u][b] += s0 * d8 * (float)(d0 + d1);
            }
        }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const float g = warp_sum(acc[0][b]), u = warp_sum(acc[1][b]);
        if (lane == 0) dst[(size_t)b * stride_dst + row] = glu_combine<dst_t>(g, u, activation);
    }
}

template <int TYPE, int B, typename dst_t>
static int launch_glu_b(const void* wg, const void* wu, const void* vy, void* dst, int K, int N, int stride_act, int stride_dst,
                        int activation, cudaStream_t s) {
    // the single-matrix plan gives the lane mapping; a stage holds the same rows of both matrices
    GemvPlan one = plan_gemv(TYPE, K, N, B, wg);
    bool ring_ok = one.staged && reinterpret_cast<uintptr_t>(wu) % 16 == 0;
    GemvGluParams p{};
    size_t smem = 0;
    if (ring_ok) {
        const int islots = 1 << one.p.log2_islots;
        const int rows_per_pass = (GEMV_CONSUMER_WARPS / one.p.warps_per_row) * (32 / islots);
        const int unit = rows_per_pass * one.p.row_align / gcd_int(rows_per_pass, one.p.row_align);
        int R = one.p.rows_per_stage / 2 / unit * unit;
        if (R < unit) R = unit;
        p.rows_per_stage = R;
        p.half_bytes = (R * one.p.row_bytes + 16 + 15) & ~15;
        p.stage_bytes = (2 * p.half_bytes + 127) & ~127;
        const int budget = runtime_info().smem_optin - 1024;
        const int wpr = one.p.warps_per_row;
        int S;
        for (S = GEMV_MAX_STAGES; S >= 2; --S) {
            const int combine = wpr > 1 ? (((S * R * wpr * 2 * B + S * R) * 4 + 127) & ~127) : 0;
            if (GEMV_BARRIER_BYTES + one.p.act_bytes + combine + S * p.stage_bytes <= budget) {
                smem = (size_t)GEMV_BARRIER_BYTES + one.p.act_bytes + combine + (size_t)S * p.stage_bytes;
                break;
            }
        }
        ring_ok = S >= 2;
        p.nstages = S;
    }
    if (!ring_ok) {
        gemv_glu_simple_kernel<TYPE, B, dst_t><<<(N + 7) / 8, 256, 0, s>>>((const uint8_t*)wg, (const uint8_t*)wu, (const uint8_t*)vy, (dst_t*)dst, K,
                                                                         N, stride_act, stride_dst, activation);
        return (int)cudaGetLastError();
    }
    p.wg = (const uint8_t*)wg;
    p.wu = (const uint8_t*)wu;
    p.act = vy;
    p.dst = dst;
    p.K = K;
    p.N = N;
    p.stride_act = stride_act;
    p.stride_dst = stride_dst;
    p.row_bytes = one.p.row_bytes;
    p.warps_per_row = one.p.warps_per_row;
    p.items_per_lane = one.p.items_per_lane;
    p.log2_wpr = one.p.log2_wpr;
    p.log2_islots = one.p.log2_islots;
    p.row_align = one.p.row_align;
    p.units_per_cta = one.p.units_per_cta;
    p.units_extra = one.p.units_extra;
    p.act_bytes = one.p.act_bytes;
    p.activation = activation;
    p.status = status_ptr();
    auto launch = [&](auto kernel) -> int {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, runtime_info().smem_optin - 1024);
        if (e != cudaSuccess) return (int)e;
        kernel<<<one.grid, GEMV_THREADS, smem, s>>>(p);
        return (int)cudaGetLastError();
    };
    // register-resident activations where the single-matrix plan has them (one or two rows of activations, one slot)
    if (one.nreg == 1 && B <= 2) return launch(gemv_glu_kernel<TYPE, B, dst_t, (B <= 2 ? 1 : 0)>);
    return launch(gemv_glu_kernel<TYPE, B, dst_t, 0>);
}

template <int TYPE, typename dst_t>
static int launch_glu(const void* wg, const void* wu, const void* vy, void* dst, int K, int N, int stride_act, int stride_dst, int b,
                      int activation, cudaStream_t s) {
    if (N <= 0 || K <= 0) return 0;
    if (K % type_block_elems(TYPE) != 0) return B200Q_ERR_INVALID;
    switch (b) {
#define B200Q_GLU_CASE(BB) \
    case BB: return launch_glu_b<TYPE, BB, dst_t>(wg, wu, vy, dst, K, N, stride_act, stride_dst, activation, s);
        B200Q_GLU_CASE(1) B200Q_GLU_CASE(2) B200Q_GLU_CASE(3) B200Q_GLU_CASE(4)
        B200Q_GLU_CASE(5) B200Q_GLU_CASE(6) B200Q_GLU_CASE(7) B200Q_GLU_CASE(8)
#undef B200Q_GLU_CASE
        default: return B200Q_ERR_UNSUPPORTED;
    }
}

int gemv_q4_k(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
int gemv_q6_k(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);
int gemv_q8_0(int, const void*, const void*, void*, int, int, int, int, int, int, const PeerExchange*, cudaStream_t);

// q, k, v: the grouped launch for one activation row, else three plain launches
template <int TYPE, typename dst_t>
static int launch_qkv(const void* wq, const void* wk, const void* wv, const void* vy, void* q_dst, void* k_dst, void* v_dst, int K, int nq, int nk,
                      int nv, int stride_act, int b, cudaStream_t s) {
    constexpr int elem = sizeof(dst_t) == 4 ? ELEM_F32 : (std::is_same<dst_t, __half>::value ? ELEM_F16 : ELEM_BF16);
    if (b == 1) {
        const int types[3] = {TYPE, TYPE, TYPE};
        const void* ws[3] = {wq, wk, wv};
        void* dsts[3] = {q_dst, k_dst, v_dst};
        const int ns[3] = {nq, nk, nv};
        const int rc = launch_gemv_group<dst_t, ACT_Q8_1>(3, types, ws, dsts, ns, K, vy, s);
        if (rc != B200Q_ERR_UNSUPPORTED) return rc;
    }
    auto one = TYPE == TYPE_Q4_K ? gemv_q4_k : (TYPE == TYPE_Q6_K ? gemv_q6_k : gemv_q8_0);
    int rc = one(elem, wq, vy, q_dst, K, nq, stride_act, nq, b, ACT_Q8_1, nullptr, s);
    if (rc == 0) rc = one(elem, wk, vy, k_dst, K, nk, stride_act, nk, b, ACT_Q8_1, nullptr, s);
    if (rc == 0) rc = one(elem, wv, vy, v_dst, K, nv, stride_act, nv, b, ACT_Q8_1, nullptr, s);
    return rc;
}

}  // namespace b200q

// The reference's symbols (crates/inference-quant/src/gguf/ffi.rs:1032-1118); void, asynchronous, allocation-free.
#define B200Q_FUSED_LAUNCHERS(tag, TYPE, etag, T)                                                                                    \
    extern "C" void launch_mmvq_gguf_##tag##_##etag##_fused_glu(const void* vx_gate, const void* vx_up, const void* vy, void* dst,       \
                                                                int ncols_x, int nrows_x, int stride_col_y, int stride_col_dst,        \
                                                                int b_size, int activation, void* stream) {                            \
        b200q::note_launch_status(b200q::launch_glu<TYPE, T>(vx_gate, vx_up, vy, dst, ncols_x, nrows_x, stride_col_y, stride_col_dst,   \
                                                             b_size, activation, (cudaStream_t)stream));                               \
    }                                                                                                                                  \
    extern "C" void launch_mmvq_gguf_##tag##_##etag##_fused_qkv(const void* vx_q, const void* vx_k, const void* vx_v, const void* vy,    \
                                                                void* q_dst, void* k_dst, void* v_dst, int ncols_x, int nrows_q,       \
                                                                int nrows_k, int nrows_v, int stride_col_y, int b_size, void* stream) { \
        b200q::note_launch_status(b200q::launch_qkv<TYPE, T>(vx_q, vx_k, vx_v, vy, q_dst, k_dst, v_dst, ncols_x, nrows_q, nrows_k,      \
                                                             nrows_v, stride_col_y, b_size, (cudaStream_t)stream));                    \
    }
#define B200Q_FUSED_TYPE(tag, TYPE)                      \
    B200Q_FUSED_LAUNCHERS(tag, TYPE, bf16, __nv_bfloat16) \
    B200Q_FUSED_LAUNCHERS(tag, TYPE, f16, __half)         \
    B200Q_FUSED_LAUNCHERS(tag, TYPE, f32, float)
B200Q_FUSED_TYPE(q8_0, b200q::TYPE_Q8_0)
B200Q_FUSED_TYPE(q4_k, b200q::TYPE_Q4_K)
B200Q_FUSED_TYPE(q6_k, b200q::TYPE_Q6_K)

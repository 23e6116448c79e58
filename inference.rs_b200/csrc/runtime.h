// Host-side state shared by the launchers: device properties, tuning knobs, and the last launch status.
#pragma once
#include <cuda_runtime.h>

namespace b200q {

// status codes of the b200q_* API (0 = ok, > 0 = a cudaError_t, < 0 = one of these)
enum : int {
    B200Q_OK = 0,
    B200Q_ERR_UNSUPPORTED = -1,   // shape / type / alignment this library has no kernel for
    B200Q_ERR_INVALID = -2,       // bad argument
    B200Q_ERR_DEVICE_STATUS = -3, // a kernel recorded a failure in the device status word
    B200Q_ERR_TOO_LARGE = -4,     // beyond a fixed capacity
};

struct RuntimeInfo {
    int sm_count;
    int smem_optin;        // max dynamic shared memory per CTA
    int smem_per_sm;       // shared memory per SM
    int use_pdl;           // launch with programmatic stream serialization
    int force_simple;      // route every GEMV to the simple kernel (testing)
    int gemv_stage_target; // bytes per shared-memory stage the GEMV planner aims at
    int gemm_direct;       // 1: the GEMM reads packed weights straight from global memory (no shared-memory staging)
    int gemv_ctas_per_sm;  // CTAs of one GEMV grid per SM: 2, or 1 to leave the other slot to the next grid
    int tc_ksplit;         // small-batch tensor-core kernel: split K over CTAs for matrices with few rows (1, testing: 0)
    int gemv_one_kernel;   // one-row GEMVs on raw activations run on the grouped kernel, so that a decode chain alternates
                           // between fewer kernels (1; 0 = the per-type kernels)
    int gemv_passes;       // decode GEMV planner: passes of all warps a stage holds (0 = the planner's own choice; 1 or 2)
    int gemv_pass_limit;   // decode GEMV planner: bytes one pass of all warps may cover before rows get more warps
    int l2_prefetch_bytes; // decode GEMV: bytes of the registered successor matrix each CTA asks L2 to fetch (0 = off;
                           // -1 = by the launch mode, see l2_prefetch_bytes_effective)
};

// With programmatic dependent launch the next launch's own CTAs start their weight stream while this launch ends, and a
// large prefetch competes with them: 64 KB measured best there, 256 KB without it.
inline int l2_prefetch_bytes_effective(const RuntimeInfo& rt) {
    return rt.l2_prefetch_bytes >= 0 ? rt.l2_prefetch_bytes : (rt.use_pdl ? 64 * 1024 : 256 * 1024);
}

// "After a launch on weight matrix w, the next launch on this stream will read matrix next_w": registered once by the
// host when it loads a model (the order of a decoder's projections is static), read by every GEMV launch. A CTA that
// has issued its last weight copy asks L2 for the first bytes of its own row range of the successor, so HBM keeps
// streaming through the tail of this launch and the gap before the next one.
struct WeightSuccessor {
    const void* w;
    int type, K, N;
};
void set_weight_successor(const void* w, const WeightSuccessor* next);  // next == nullptr: forget w
void clear_weight_successors();
bool find_weight_successor(const void* w, WeightSuccessor* out);

const RuntimeInfo& runtime_info();
RuntimeInfo& runtime_info_mut();
unsigned int* status_ptr();          // device address of the status word of the current device (cached)
// diagnostics: when a trace buffer is set, every GEMV launch gets the next 32-slot record of it (wrapping)
void set_trace_buffer(unsigned long long* dev, int records);
unsigned long long* trace_slot();
unsigned long long* trace_buffer(int* slots);

// cudaFuncAttributeMaxDynamicSharedMemorySize belongs to a (function, device) pair: launchers set it once per device
// and kernel instantiation, on the first launch there (one static PerDeviceOnce per instantiation).
struct PerDeviceOnce {
    bool done[64] = {};
    template <typename Fn> cudaError_t run(Fn&& fn) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= 64) return fn();
        if (!done[dev]) {
            e = fn();
            if (e != cudaSuccess) return e;
            done[dev] = true;
        }
        return cudaSuccess;
    }
};

int note_launch_status(int status);  // remembers the first non-zero status; returns its argument
int take_launch_status();            // returns and clears it

}  // namespace b200q

// Host-side state shared by the launchers (see runtime.h).
#include "runtime.h"

#include <atomic>
#include <cstdlib>
#include <mutex>
#include <shared_mutex>
#include <unordered_map>

namespace b200q {

__device__ unsigned int g_status_word[4] = {0, 0, 0, 0};

static RuntimeInfo g_rt = {0, 0, 0, 0, 0, 40 * 1024, 0, 1, 1, 1, 0, 48 * 1024, -1};
static std::atomic<int> g_launch_status{0};

static void query_device() {
    int dev = 0;
    int sm = 0, optin = 0, per_sm = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) {
        cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
    } else {
        cudaGetLastError();
    }
    // B200 values when no device can be asked (planning on a CPU-only host)
    g_rt.sm_count = sm > 0 ? sm : 148;
    g_rt.smem_optin = optin > 0 ? optin : 227 * 1024;
    g_rt.smem_per_sm = per_sm > 0 ? per_sm : 228 * 1024;
    if (const char* e = std::getenv("B200Q_PDL")) g_rt.use_pdl = std::atoi(e);
    if (const char* e = std::getenv("B200Q_GEMV_STAGE_BYTES")) {
        int v = std::atoi(e);
        if (v >= 1024) g_rt.gemv_stage_target = v;
    }
    if (const char* e = std::getenv("B200Q_L2_PREFETCH_BYTES")) g_rt.l2_prefetch_bytes = std::atoi(e) & ~15;
}

RuntimeInfo& runtime_info_mut() {
    if (g_rt.sm_count == 0) query_device();
    return g_rt;
}
const RuntimeInfo& runtime_info() { return runtime_info_mut(); }

unsigned int* status_ptr() {
    static unsigned int* cached[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        cached[dev] = static_cast<unsigned int*>(p);
    }
    return cached[dev];
}

static unsigned long long* g_trace = nullptr;
static int g_trace_records = 0;
static std::atomic<int> g_trace_next{0};
void set_trace_buffer(unsigned long long* dev, int records) {
    g_trace = dev;
    g_trace_records = records;
    g_trace_next = 0;
}

unsigned long long* trace_buffer(int* slots) {
    *slots = g_trace ? g_trace_records * 32 : 0;
    return g_trace;
}
unsigned long long* trace_slot() {
    if (g_trace == nullptr || g_trace_records <= 0) return nullptr;
    const int i = g_trace_next.fetch_add(1) % g_trace_records;
    return g_trace + (size_t)i * 32;
}

static std::shared_mutex g_succ_mutex;
static std::unordered_map<const void*, WeightSuccessor> g_successors;
void set_weight_successor(const void* w, const WeightSuccessor* next) {
    std::unique_lock<std::shared_mutex> lock(g_succ_mutex);
    if (next == nullptr || next->w == nullptr) g_successors.erase(w);
    else g_successors[w] = *next;
}
void clear_weight_successors() {
    std::unique_lock<std::shared_mutex> lock(g_succ_mutex);
    g_successors.clear();
}
bool find_weight_successor(const void* w, WeightSuccessor* out) {
    std::shared_lock<std::shared_mutex> lock(g_succ_mutex);
    if (g_successors.empty()) return false;
    auto it = g_successors.find(w);
    if (it == g_successors.end()) return false;
    *out = it->second;
    return true;
}

int note_launch_status(int status) {
    if (status != 0) {
        int expected = 0;
        g_launch_status.compare_exchange_strong(expected, status);
    }
    return status;
}
int take_launch_status() { return g_launch_status.exchange(0); }

}  // namespace b200q

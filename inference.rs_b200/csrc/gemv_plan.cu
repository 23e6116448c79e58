// Planner introspection for the decode GEMV (kept out of the per-type instance files).
#include "gemv_impl.cuh"

namespace b200q {
void gemv_describe(int type, int K, int N, int b, int* out) {
    GemvPlan plan = plan_gemv(type, K, N, b, nullptr);
    out[0] = plan.staged;
    out[1] = plan.grid;
    out[2] = (int)plan.smem;
    out[3] = plan.p.nstages;
    out[4] = plan.p.rows_per_stage;
    out[5] = plan.p.warps_per_row;
    out[6] = plan.p.stage_bytes;
    out[7] = plan.p.row_align;
    out[8] = plan.p.items_per_lane;
    out[9] = plan.nreg;
}
}  // namespace b200q

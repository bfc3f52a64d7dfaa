#include "qgemv_common.cuh"
namespace qgemv {
MmaPlan plan_mma(const qgemv_problem&) { return MmaPlan{false, 1, 0, 0, nullptr}; }
int launch_mma(const Args&, int, bool, const MmaPlan&, cudaStream_t) { set_error("mma kernel not built"); return QGEMV_ERR_LAUNCH; }
}

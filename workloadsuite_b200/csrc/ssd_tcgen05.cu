// tcgen05 / TMEM chunked SSD kernel (placeholder until the kernel lands).
#include "ssd_common.cuh"

namespace ssd {
bool tc_supports(const SsdArgs&) { return false; }
int tc_default_segments(const SsdArgs&) { return 1; }
int launch_tc(const SsdArgs&, const ScanParams&, cudaStream_t) { return SSD_ERR_UNSUPPORTED; }
}  // namespace ssd

// placeholder until the tcgen05 kernel lands
#include "w4a16_common.cuh"
namespace kiln {
bool prefill_supported(int, int, int, int) { return false; }
size_t prefill_workspace_bytes(int, int, int) { return 0; }
int launch_prefill(const GemmArgs &) { return KILN_W4A16_ERR_KERN_SHAPE; }
}  // namespace kiln

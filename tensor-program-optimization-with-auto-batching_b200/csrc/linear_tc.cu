// placeholder until the tcgen05 kernel lands
#include "linear.cuh"
namespace mlora {
bool linear_tc_supported(const LinearArgs&) { return false; }
size_t linear_tc_workspace(int, int, int) { return 0; }
int launch_linear_tc(const LinearArgs&, void*, size_t, cudaStream_t) { return fail(MLORA_EINVAL, "no tc kernel"); }
}  // namespace mlora

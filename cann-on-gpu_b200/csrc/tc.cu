#include "kernels.h"
namespace qmm {
bool tc_supported(const MatmulArgs &) { return false; }
void tc_plan(MatmulArgs &p) { p.split_k = 1; }
uint64_t tc_workspace_bytes(const MatmulArgs &) { return 0; }
cudaError_t launch_tc(const MatmulArgs &, cudaStream_t) { return cudaErrorNotSupported; }
}

// placeholder until the low-rank stages land
#include "bsq_internal.hpp"
namespace bsq {
SvdWorkspace *svd_workspace_create(int, int, int, int, int) { return nullptr; }
void svd_workspace_destroy(SvdWorkspace *) {}
cudaError_t svd_lowrank(SvdWorkspace *, const float *, float *, float *, float *, unsigned long long, unsigned *, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t reconstruct_lowrank(const float *, const float *, const float *, int, int, int, const float *, float *, unsigned *, int, cudaStream_t) { return cudaErrorNotSupported; }
}

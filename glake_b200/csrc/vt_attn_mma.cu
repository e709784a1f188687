// Placeholder translation unit: tensor-core GQA variant (filled in next).
#include "../../include/vtensor.h"
#include "vt_kernels.h"
namespace vt {
int launch_attn_mma(const AttnParams &, int, cudaStream_t) { return VT_ERR_UNSUPPORTED; }
}  // namespace vt

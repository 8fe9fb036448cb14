// Tensor-core LUT decode kernel (placeholder until the mma path lands).
#include "tq4_attention.cuh"
namespace tq4 {
bool attention_mma_supported(const AttnShape&, int) { return false; }
int launch_attention_mma(const AttnArgs&, cudaStream_t) { return TQ4_ERR_UNSUPPORTED; }
}  // namespace tq4

// Tensor-core decode attention for head_dim 128 (placeholder until the kernel
// lands: nothing is eligible, every call takes the scalar kernel).
#include "attention_common.cuh"

namespace jpt {
bool attention_mma_eligible(const jpt_attn_params&) { return false; }
int attention_mma_pick_splits(const jpt_attn_params&) { return 1; }
int launch_attention_mma(const jpt_attn_params&, const AttnArgs&, cudaStream_t) {
  return fail(JPT_EINVAL, "flash_decode: tensor-core kernel not built");
}
}  // namespace jpt

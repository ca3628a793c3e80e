// The reference's own call shape (one residual vector against flat caches of `pos` rows per layer) run as pos + 1
// attention rows of which the last is live: buffers and the forward shared by its reverse and forward modes.
#pragma once

#include <vector>

#include "plan.cuh"

namespace b200 {

struct TokLayer {
  float* x_in; void* xb; float* rinv1; void* qkv; void* o; float* lse;
  float* x_mid; void* xb2; float* rinv2; void* gate; void* up; void* hg;
};
struct TokWs {
  std::vector<TokLayer> layer;
  float* x_last; float* rinv_f;
  float* dx; void* dxb; void* dhg; void* dgu; void* d_o; void* dqkv; float* delta; float* dg_part;
  void* splitk; size_t splitk_bytes;
  int n_parts;
};

// Carves the buffers of a step over S = pos + 1 attention rows; with a null arena base it only counts.
void carve_token(const B200Plan& p, Arena& a, int S, TokWs* w);
size_t token_vjp_workspace_bytes(const B200Plan& p, int pos);
// Forward keeping the activations in `t`; `hidden` receives the final-normed hidden state (fp32 [d]).
int32_t token_forward_run(B200Plan* p, const TokWs& t, const float* x, const void* key_cache, const void* value_cache,
                          int pos, const uint8_t* w, const PackedLayout& wl, float* hidden, cudaStream_t stream);

}  // namespace b200

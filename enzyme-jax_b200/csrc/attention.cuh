// Attention kernels of the llama path: causal prefill/training forward and
// backward, and decode over the paged KV cache.
#pragma once

#include "common.cuh"

namespace b200 {

// q,k,v,o are [batch*seq, ld] row-major with heads side by side in a row
// (head h occupies columns h*head_size .. +head_size).
struct AttnArgs {
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  void* o = nullptr;
  float* lse = nullptr;  // [batch, n_heads, seq] or null
  int batch = 0, seq = 0, n_heads = 0, head_size = 0;
  int ldq = 0, ldkv = 0, ldo = 0;
  int dtype = B200_BF16;
};

int32_t launch_attn_fwd_simt(const AttnArgs& a, cudaStream_t stream);
int32_t launch_attn_fwd_mma(const AttnArgs& a, cudaStream_t stream);
bool attn_fwd_mma_supports(const AttnArgs& a);
// impl: 0 = pick, 1 = tensor-core kernel, 2 = CUDA-core kernel
int32_t launch_attn_fwd(const AttnArgs& a, int impl, cudaStream_t stream);

// Backward.  dq,dk,dv have the layout of q,k,v; d_o that of o.
struct AttnBwdArgs {
  AttnArgs f;              // forward tensors (q,k,v,o,lse)
  const void* d_o = nullptr;
  void* dq = nullptr;
  void* dk = nullptr;
  void* dv = nullptr;
  int lddq = 0, lddkv = 0, lddo = 0;
  float* delta = nullptr;  // scratch [batch, n_heads, seq]: rowsum(dO * O)
};
int32_t launch_attn_bwd_simt(const AttnBwdArgs& a, cudaStream_t stream);
int32_t launch_attn_bwd_tc(const AttnBwdArgs& a, cudaStream_t stream);
bool attn_bwd_tc_supports(const AttnBwdArgs& a);
// delta[b,h,t] = sum_e dO[t,e] * O[t,e]  (first step of either backward)
int32_t launch_attn_delta(const AttnBwdArgs& a, cudaStream_t stream);
// impl: 0 = pick, 1 = tensor-core kernels, 2 = CUDA-core kernels
int32_t launch_attn_bwd(const AttnBwdArgs& a, int impl, cudaStream_t stream);

// Decode: one query row per (sequence, head) against `ctx` cached rows held in
// pages.  The context is split into chunks handled by different CTAs; partial
// (max, sum, acc) go to scratch and a second kernel combines them.
struct AttnDecodeArgs {
  const void* q = nullptr;        // [batch, ldq]
  const void* kv_pages = nullptr; // layer base: K pages at [0], V pages at [1]: [2, n_pages, n_heads, page_size, head_size]
  const int32_t* page_table = nullptr;  // [batch, max_pages]
  void* o = nullptr;              // [batch, ldo]
  float* scratch = nullptr;       // decode_scratch_floats() floats
  int batch = 0, ctx = 0, n_heads = 0, head_size = 0;
  int ldq = 0, ldo = 0;
  int n_pages = 0, page_size = 0, max_pages = 0;
  int d_local = 0;                // row width of a page (n_heads * head_size)
  int dtype = B200_BF16;
  int n_splits = 0;
};
size_t decode_scratch_floats(int batch, int n_heads, int head_size, int n_splits);
int decode_pick_splits(int batch, int n_heads, int ctx);
int32_t launch_attn_decode(const AttnDecodeArgs& a, cudaStream_t stream);

}  // namespace b200

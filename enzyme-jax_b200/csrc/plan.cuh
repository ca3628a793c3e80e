// Launch plan of the llama path: shapes, tensor-parallel shard sizes, the layout
// of the packed weight / gradient buffers, and the carving of the caller's
// workspace and saved-activation buffers.
#pragma once

#include <stddef.h>

#include <vector>

#include "common.cuh"

namespace b200 {

struct LayerOffsets {
  size_t wqkv, wo, w13, w2;          // byte offsets of the matrices
  size_t wqkv_t, wo_t, w13_t, w2_t;  // transposed copies (weights only)
};

struct PackedLayout {
  size_t g_att = 0, g_ffn = 0, g_final = 0;  // fp32 gains
  size_t emb = 0;
  std::vector<LayerOffsets> layer;
  size_t wcls = 0, wcls_t = 0;
  size_t total = 0;
};

// Carves consecutive 256-byte aligned regions out of a caller buffer; with a
// null base it only counts.
struct Arena {
  uint8_t* base;
  size_t used = 0;
  explicit Arena(void* b) : base(reinterpret_cast<uint8_t*>(b)) {}
  template <typename T = void> T* take(size_t bytes) {
    T* p = base ? reinterpret_cast<T*>(base + used) : nullptr;
    used += align_up(bytes, 256);
    return p;
  }
};

// Activations of one layer: slices of the saved buffer when the forward keeps
// them for the backward pass, else workspace regions shared by all layers.
struct LayerActs {
  float* x_in = nullptr;   // [T,d] residual stream entering the layer
  void* xb = nullptr;      // [T,d] normed input of the attention block
  float* rinv1 = nullptr;  // [T]
  void* qkv = nullptr;     // [T,3*d_loc] rotated q,k and v
  void* o = nullptr;       // [T,d_loc] attention output
  float* lse = nullptr;    // [B,H_loc,S]
  float* x_mid = nullptr;  // [T,d] residual stream after attention
  void* xb2 = nullptr;     // [T,d]
  float* rinv2 = nullptr;  // [T]
  void* gate = nullptr;    // [T,h_loc]
  void* up = nullptr;      // [T,h_loc]
  void* hg = nullptr;      // [T,h_loc]
  float* x_out = nullptr;  // [T,d] residual stream leaving the layer
};
struct FinalActs {
  float* x_last = nullptr;
  float* rinv_f = nullptr;
  void* xf = nullptr;
};
struct FwdActs {
  std::vector<LayerActs> layer;
  FinalActs fin;
};

}  // namespace b200

struct B200Plan {
  B200LlamaConfig cfg;
  int tp_rank = 0, tp_size = 1;
  void* comm = nullptr;
  int d = 0, h = 0, L = 0, H = 0, hs = 0, V = 0;
  int d_loc = 0, h_loc = 0, V_loc = 0, H_loc = 0;
  int esize = 2;
  int dtype = B200_BF16;
  int device = 0;
  int gemm_impl = 0, attn_impl = 0;
  // tensor parallelism: the all-reduces run on a stream of their own, chunk by chunk, while the
  // projection of the next chunk computes; `reserve_sms` SMs are left to the collective's kernels
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_fork[8] = {}, ev_join[8] = {};
  int reserve_sms = 0;
  int tp_chunks = 1;
  bool tp_bands = true;      // column-parallel GEMMs wait for the gathered rows band by band instead of the exchange kernel
  bool tp_push = true;       // row-parallel GEMMs store their partial product straight into the owners' memory
  int tp_bands_last = 0;     // whether the last tensor-parallel forward consumed the gathered rows band by band
  int tp_push_last = 0;      // whether the last tensor-parallel forward did so (it needs shapes the CTA-pair GEMM takes)
  bool tp_pipeline = false;  // ... and runs two halves of the batch so that one half's exchange overlaps the other's compute
  bool row_shard = true;  // tensor-parallel prefill keeps T/tp residual rows per rank when peer memory is up
  float* rope_cos = nullptr;  // [seq_len, hs/2], owned by the plan
  float* rope_sin = nullptr;
  b200::PackedLayout wl;   // weights
  b200::PackedLayout wlt;  // weights followed by transposed copies
  b200::PackedLayout gl;   // gradients (everything fp32)
};

namespace b200 {

void build_layout(const B200Plan& p, size_t mat_esize, bool with_t, PackedLayout* out);
// Carves the activations of a forward over T = B*S tokens.  keep: per-layer
// buffers (the saved-activation layout); otherwise one shared set.
void carve_forward(const B200Plan& p, Arena& a, int B, int S, bool keep, FwdActs* out);

int32_t comm_allreduce(void* comm, void* data, size_t count, int dtype, cudaStream_t stream);
// This rank's peer-mapped exchange buffer when the peer path is up and `bytes` fit, else null.
void* comm_peer_buffer(void* comm, size_t bytes);
// out = resid + sum over ranks of the `count` elements each rank left in its exchange buffer
int32_t comm_peer_allreduce_add(void* comm, size_t count, int dtype, const float* resid, float* out,
                                cudaStream_t stream);

// Row-sharded prefill: the two regions of this rank's exchange buffer (partial product, gathered activations) when
// the peer path is up and both fit; comm_peer_reduce_norm sums the partials of this rank's T / world rows over the
// ranks, adds them to x_own (fp32 [T / world, d], in place; skipped when !reduce), and leaves gain * x * rinv of those
// rows in every rank's gathered-activation region.  Its completion means the region of this rank is whole.
bool comm_peer_rowshard_buffers(void* comm, size_t bytes_each, void** part, void** xb);
// pushed: the partial products were stored by the producing GEMM straight into their owners' memory
// (comm_peer_push_bases + GemmArgs::push_rows), so the kernel sums them from this rank's own slots.
// bands: when given, the kernel does NOT end by waiting for the peers' rows; it returns as soon as this rank's rows
// are delivered and *bands says how the consumer can wait band by band itself (GemmArgs::band_flags): flags[o]
// reaches `epoch` once rank o's rows are whole in this rank's gathered region.
struct PeerBands {
  const uint32_t* flags = nullptr;
  uint32_t epoch = 0;
  int rows = 0, first = 0;
  long long budget = 0;
};
int32_t comm_peer_reduce_norm(void* comm, int T, int d, int dtype, bool reduce, float* x_own, const float* gain,
                              float eps, cudaStream_t stream, bool pushed = false, PeerBands* bands = nullptr);
int32_t comm_peer_reduce_norm_at(void* comm, int T, int d, int dtype, bool reduce, float* x_own, const float* gain,
                                 float eps, size_t part_rel, size_t xb_rel, bool lean, cudaStream_t stream,
                                 bool pushed = false, PeerBands* bands = nullptr);
bool comm_peer_push_bases(void* comm, int T, int d, int dtype, void** bases);
int32_t launch_peer_wait_selftest(long long budget, uint32_t* reached_end, cudaStream_t stream);

// Environment knobs (read once at plan creation): B200_GEMM_IMPL and
// B200_ATTN_IMPL select 0 = pick, 1 = tensor-core kernels, 2 = CUDA-core kernels.
int env_int(const char* name, int dflt);

}  // namespace b200

// Memory-bound kernels of the llama path: embedding gather, RMSNorm, residual
// add, layout/dtype conversion, and their backward counterparts.
#pragma once

#include "common.cuh"

namespace b200 {

// x[t, :] = table[tokens[t], :] as fp32 (residual stream).  test/llama.py:109-113.
int32_t launch_embed(const int32_t* tokens, const void* table, int table_dtype, float* x, int n_tokens, int dim,
                     int vocab, cudaStream_t stream);

// y = gain * x * rsqrt(mean(x^2) + eps) per row; rinv (optional) receives the
// per-row factor.  test/llama.py:6-10.
int32_t launch_rmsnorm(const float* x, const float* gain, void* y, float* rinv, int rows, int dim, float eps,
                       int out_dtype, cudaStream_t stream);

// x[i] += delta[i] (delta of dtype `dtype`), the residual add after a
// tensor-parallel all-reduce.
int32_t launch_add_to_f32(float* x, const void* delta, int dtype, size_t n, cudaStream_t stream);

// dst[map(r), c] = src[r, c] with dtype conversion, where
// map(r) = (r / group) * group_stride + group_offset + r % group.
int32_t launch_copy_rows(const void* src, int src_dtype, int src_ld, void* dst, int dst_dtype, int dst_ld, int rows,
                         int cols, int group, int group_stride, int group_offset, cudaStream_t stream);

// dst[c, r] = src[r, c] with dtype conversion.
int32_t launch_transpose(const void* src, int src_dtype, int src_ld, void* dst, int dst_dtype, int dst_ld, int rows,
                         int cols, cudaStream_t stream);

// Position tables cos/sin[pos, j] for j < head_size/2 (test/llama.py:127-140).
int32_t launch_rope_table(float* cos_t, float* sin_t, int n_pos, int head_size, float theta, cudaStream_t stream);

// ---- backward ---------------------------------------------------------------

// RMSNorm backward for y = g * x * r: dx (+)= r*u - x * r^3/d * sum(u*x), u = g*dy;
// dgain partials are written per CTA to `dg_part` [n_parts, dim] and reduced by
// launch_colsum_parts (fixed order, no atomics).  dy has dtype `dy_dtype`.  dx_copy (optional, dtype of dy, may be dy
// itself) receives the updated dx as well: the next GEMMs take it as their low-precision operand.
int32_t launch_rmsnorm_bwd(const float* x, const float* gain, const float* rinv, const void* dy, int dy_dtype,
                           float* dx, int accumulate_dx, void* dx_copy, float* dg_part, int n_parts, int rows, int dim,
                           cudaStream_t stream);
int rmsnorm_bwd_parts(int rows);
// out[c] (+)= sum_p part[p, c]
int32_t launch_colsum_parts(const float* part, int n_parts, int dim, float* out, int accumulate,
                            cudaStream_t stream);

// Rotates adjacent pairs of the first rope_cols columns by the NEGATIVE angle
// (adjoint of the forward rotation), in place.
int32_t launch_rope_bwd(void* dqkv, int dtype, int ld, int rows, int rope_cols, int head_size, int seq_len,
                        const float* cos_t, const float* sin_t, cudaStream_t stream);

// SwiGLU backward: given gate a, up b, dh -> d(gate|up) in the interleaved
// column layout of the fused W1/W3 GEMM output ([8 gate | 8 up] per 16 columns).
int32_t launch_swiglu_bwd(const void* gate, const void* up, const void* dh, void* dgu, int dtype, int rows,
                          int hidden, cudaStream_t stream);

// dtable[tokens[t], :] += dx[t, :], deterministic (tokens are bucketed per row
// of the table by a sort-free two-pass scheme: one thread block per vocabulary
// slice scans the token list in order).
int32_t launch_embed_bwd(const int32_t* tokens, const float* dx, float* dtable, int n_tokens, int dim, int vocab,
                         cudaStream_t stream);

// out = (TOut) in, elementwise.
int32_t launch_convert(const void* src, int src_dtype, void* dst, int dst_dtype, size_t n, cudaStream_t stream);

// x[i] = 0
int32_t launch_zero_f32(float* x, size_t n, cudaStream_t stream);

// out[r] = argmax of row r (lowest index among equal maxima): greedy sampling from fp32 logits
int32_t launch_argmax_rows(const float* x, int rows, int cols, int ld, int32_t* out, cudaStream_t stream);

}  // namespace b200

/* C ABI of the B200-native llama forward / VJP path.
 *
 * This is the boundary an XLA typed-FFI handler (api_version 4) binds to.  The
 * reference registers such handlers with
 *   Ffi::Bind().Ctx<PlatformStream<CUstream>>().Attr<T>(..).Arg<AnyBuffer>()..Ret<AnyBuffer>()
 * (src/enzyme_ad/jax/xla_ffi/cuda/blas.cc:286-314) and
 *   XLA_FFI_REGISTER_HANDLER(GetXlaFfiApi(), name, "CUDA", handler)
 * (src/enzyme_ad/jax/xla_ffi/register.cc:21-27).  Each entry point below is
 * what such a handler calls after unpacking its buffers: plain device pointers,
 * sizes, a stream; no framework types.
 *
 * Conventions (matching the reference's handler rules):
 *  - the caller owns every buffer, outputs and scratch included
 *    (primitives.py:712-727 appends an i8[tmpBuf] result as scratch);
 *  - work is enqueued on the given stream and the call returns without
 *    synchronising (gpu.cc:122-125,153);
 *  - the return value is a status code, 0 on success; b200_last_error() gives
 *    the thread-local message (the handler maps it to ffi::Error, as
 *    blas.cc:80-115 does for cuBLAS failures).
 *  - nothing here falls back to a CPU implementation.
 */
#ifndef B200_LLAMA_H_
#define B200_LLAMA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_API __attribute__((visibility("default")))

typedef void* b200_stream_t; /* cudaStream_t / CUstream */

enum B200Status {
  B200_OK = 0,
  B200_ERR_INVALID_ARG = 1,   /* null pointer, negative size */
  B200_ERR_BAD_SHAPE = 2,     /* shape the kernels do not cover */
  B200_ERR_BAD_DTYPE = 3,
  B200_ERR_MISALIGNED = 4,    /* pointer or stride not 16-byte aligned */
  B200_ERR_WORKSPACE = 5,     /* workspace smaller than b200_workspace_bytes */
  B200_ERR_ARCH = 6,          /* device is not sm_100 */
  B200_ERR_CUDA = 7,
  B200_ERR_NCCL = 8,
  B200_ERR_TIMEOUT = 9,       /* a bounded device-side wait ran out */
  B200_ERR_UNSUPPORTED = 10
};

enum B200DType { B200_F32 = 0, B200_BF16 = 1 };

/* Model description: the keys of the reference's config dict
 * (test/llama.py:246-254) plus the numeric type and the two constants the
 * reference hard-codes (theta at test/llama.py:129, eps at :9). */
typedef struct B200LlamaConfig {
  int32_t dim;
  int32_t hidden_dim;
  int32_t n_layers;
  int32_t n_heads;
  int32_t n_kv_heads; /* must equal n_heads, as in the reference (test/llama.py:162) */
  int32_t vocab_size;
  int32_t seq_len;    /* maximum sequence length */
  int32_t dtype;      /* B200DType of weights and activations; accumulation, the
                         residual stream, logits and gradients are always fp32 */
  float rope_theta;
  float rms_eps;
} B200LlamaConfig;

typedef struct B200Plan B200Plan;

/* Order of the weight leaves everywhere in this ABI: the sorted key order in
 * which JAX flattens the reference's weight dict (primitives.py:1537-1569
 * flattens args with tree_flatten), with the embedding leaf the reference
 * names at test/llama.py:109-112 in its sorted place. */
enum B200Leaf {
  B200_LEAF_RMS_ATT = 0,   /* [L, d]        */
  B200_LEAF_RMS_FFN = 1,   /* [L, d]        */
  B200_LEAF_RMS_FINAL = 2, /* [d]           */
  B200_LEAF_TOK_EMB = 3,   /* [V, d]        */
  B200_LEAF_W1 = 4,        /* [L, h, d]     */
  B200_LEAF_W2 = 5,        /* [L, d, h]     */
  B200_LEAF_W3 = 6,        /* [L, h, d]     */
  B200_LEAF_WCLS = 7,      /* [V, d]        */
  B200_LEAF_WK = 8,        /* [L, d, d]     */
  B200_LEAF_WO = 9,        /* [L, d, d]     */
  B200_LEAF_WQ = 10,       /* [L, d, d]     */
  B200_LEAF_WV = 11,       /* [L, d, d]     */
  B200_NUM_LEAVES = 12
};

/* ---- library / device ---------------------------------------------------- */

/* Thread-local message of the last failing call on this thread.  Replaces the
 * ffi::Error text of xla_ffi/cuda/blas.cc:80-115. */
B200_API const char* b200_last_error(void);

/* Version string "major.minor". */
B200_API const char* b200_version(void);

/* Reads and clears the device-side status word that kernels with bounded
 * waits set when a wait runs out.  Synchronises the stream (the one place that
 * does, like xla_throw_error in xla_ffi/cuda/throw_error.cc:20-31).  Returns
 * B200_OK or B200_ERR_TIMEOUT; *code receives the raw word. */
B200_API int32_t b200_device_status(b200_stream_t stream, uint32_t* code);

/* Greedy sampling on the device: out_tokens[r] = argmax of the r-th row of fp32 logits [rows, ld] (first `cols`
 * columns; the lowest index among equal maxima).  The decode loop feeds out_tokens straight back into
 * b200_decode_step, so no logits leave the GPU.  The reference leaves sampling to its caller (test/llama.py returns the
 * hidden state); this is the device-side half of the decode loop the serving configuration needs. */
B200_API int32_t b200_argmax(const float* logits, int32_t rows, int32_t cols, int32_t ld, int32_t* out_tokens,
                             b200_stream_t stream);

/* Failure-detection self-test: launches one CTA that waits, with a budget of budget_cycles SM
 * clocks, on an mbarrier nothing ever signals.  The wait gives up, the kernel writes 1 to
 * *reached_end_device and returns, and the next b200_device_status call answers
 * B200_ERR_TIMEOUT; the context stays usable.  This is the host-visible form of the bounded
 * waits every tcgen05 kernel of the library uses (the reference has no counterpart: its
 * failures surface as XLA errors, xla_ffi/cuda/throw_error.cc:20-35). */
B200_API int32_t b200_selftest_bounded_wait(int64_t budget_cycles, uint32_t* reached_end_device, b200_stream_t stream);

/* The same self-test for the waits on OTHER ranks (the flags that tensor-parallel kernels poll in peer-mapped
 * memory): one CTA waits, for budget_cycles SM clocks, on peer flags that nothing sets.  The wait gives up,
 * *reached_end_device receives 1, the next b200_device_status call answers B200_ERR_TIMEOUT, and the context stays
 * usable.  Needs no second GPU and no communicator.  The budget of the real kernels is B200_PEER_WAIT_MCYCLES
 * (millions of SM clocks, default 4000, read at b200_comm_init_rank). */
B200_API int32_t b200_selftest_peer_wait(int64_t budget_cycles, uint32_t* reached_end_device, b200_stream_t stream);

/* Number of kernels this library has launched in this process. */
B200_API int64_t b200_launch_count(void);

/* Per-kernel timing with CUDA events on the launching stream, the counterpart
 * of the reference's profiler-based step timing (test/xprof_utils.py:71-157).
 * b200_profile_enable(1) clears earlier samples and brackets every GEMM and
 * attention launch with an event pair; b200_profile_read synchronises those
 * events and returns, for one kernel class (0 single-CTA tcgen05 GEMM gemm_tc_kernel, 1 FFMA GEMM,
 * 2 attention forward, 3 attention backward, 4 decode attention, 5 exchange between ranks,
 * 6 CTA-pair tcgen05 GEMM gemm_tc2_kernel), the summed
 * milliseconds, the summed algorithmic work (flops; bytes for classes 4 and 5) and
 * the launch count.  Off by default; costs two event records per launch. */
B200_API int32_t b200_profile_enable(int32_t on);
B200_API int32_t b200_profile_read(int32_t kernel_class, double* total_ms, double* total_work, int64_t* launches);

/* ---- plan ---------------------------------------------------------------- */

/* Creates the launch plan for one model on the current device.  tp_size > 1
 * shards heads, hidden units and vocabulary rows Megatron-style over the ranks
 * of `comm` (a handle from b200_comm_init_rank, or NULL when tp_size == 1).
 * Replaces the compile step the reference performs for a jitted function
 * (primitives.py:536-783: lowering + pass pipeline); there is no IR here, the
 * plan is the fixed kernel sequence for this model. */
B200_API int32_t b200_plan_create(const B200LlamaConfig* cfg, int32_t tp_rank, int32_t tp_size,
                                  void* comm, B200Plan** out);
B200_API int32_t b200_plan_destroy(B200Plan* plan);

/* The plan for (config, tensor-parallel rank/size, communicator) on the current device from a process-wide registry:
 * created on first use, shared afterwards, destroyed at process exit.  This is what a custom-call handler uses, which
 * is handed attributes and buffers on every call and has no place to keep a handle; it stands for the reference's
 * registry of compiled kernels keyed by an identifier (enzyme_call.cc:173,263,282: a map behind a reader/writer
 * lock).  Safe to call from several threads; plans are immutable after creation apart from b200_plan_set_option, which
 * a caller sharing a plan between threads must not call while another thread launches through it. */
B200_API int32_t b200_plan_cached(const B200LlamaConfig* cfg, int32_t tp_rank, int32_t tp_size, void* comm,
                                  B200Plan** out);

/* Run-time options of a plan, by name.  "tp_pipeline": 1 = the tensor-parallel prefill (b200_forward with tp_size > 1
 * over peer memory) runs two halves of the batch so that one half's exchange crosses NVLink beside the other half's
 * GEMMs and attention, 0 = one batch with the exchange between the kernels (the default, unless the B200_TP_PIPELINE
 * environment variable says 1).  Every rank of the communicator must hold the same value whenever
 * b200_forward runs.  Results do not depend on it.  "tp_push": 1 (default, or B200_TP_PUSH) = the row-parallel
 * projections (Wo, W2) of that prefill store every band of rows of their partial product straight into the memory of
 * the rank that owns the rows, tile by tile while the GEMM computes, and the exchange kernel sums from local memory;
 * 0 = they store locally and the exchange kernel pulls over NVLink; same value on every rank.  "tp_push_last"
 * (get only): whether the last forward did push (it needs shapes the CTA-pair GEMM takes and T / tp_size a multiple
 * of 32).  "tp_bands": 1 (default, or B200_TP_BANDS) = the exchange kernel returns once this rank's rows are
 * delivered and the column-parallel projection that follows (QKV, W1|W3, logits) starts on those rows and waits, with
 * a bounded wait, for every other rank's band of rows just before it first loads from it, 0 = the exchange kernel
 * waits for all ranks; same value on every rank; "tp_bands_last" (get only) as above.  Unknown names:
 * B200_ERR_INVALID_ARG.  The reference has no
 * counterpart (its options travel as pass-pipeline strings, primitives.py:56-115). */
B200_API int32_t b200_plan_set_option(B200Plan* plan, const char* name, int32_t value);
B200_API int32_t b200_plan_get_option(const B200Plan* plan, const char* name, int32_t* value);

/* Bytes of the packed weight buffer for this rank; with_transposed != 0 adds
 * the transposed copies the backward pass contracts against. */
B200_API int32_t b200_packed_weight_bytes(const B200Plan* plan, int32_t with_transposed, size_t* bytes);

/* Packs the 12 leaves (device pointers, B200Leaf order, element type
 * leaf_dtype, full unsharded shapes) into the layout the kernels read:
 * Wq/Wk/Wv rows concatenated, W1/W3 rows interleaved in groups of 8, this
 * rank's shard only.  Stands in for the layout assignment XLA performs on the
 * custom call's operand_layouts (Passes/LowerEnzymeXLABLAS.cpp:463-479). */
B200_API int32_t b200_pack_weights(const B200Plan* plan, const void* const* leaves, int32_t leaf_dtype,
                                   int32_t with_transposed, void* packed, b200_stream_t stream);

/* mode: 0 forward (inference), 1 forward keeping activations for backward,
 * 2 backward, 3 decode step. */
B200_API int32_t b200_workspace_bytes(const B200Plan* plan, int32_t mode, int32_t batch, int32_t seq, size_t* bytes);
B200_API int32_t b200_saved_bytes(const B200Plan* plan, int32_t batch, int32_t seq, size_t* bytes);

/* ---- forward / backward / decode ----------------------------------------- */

/* Full causal forward (the reference's `forward`, test/llama.py:35-238,
 * applied to every position of `batch` sequences, with the embedding lookup
 * and the logits projection of test/llama.py:109-113,236 enabled).
 *   tokens  int32 [batch, seq]
 *   logits  fp32  [batch*seq, vocab/tp_size]  (this rank's vocabulary rows)
 *   saved   NULL, or b200_saved_bytes() bytes that receive the activations
 *           b200_backward needs
 *   kv_out  NULL, or [L, 2, batch, seq, d/tp] receiving rotated K and V */
B200_API int32_t b200_forward(B200Plan* plan, const int32_t* tokens, int32_t batch, int32_t seq,
                              const void* packed_w, float* logits, void* saved, void* kv_out,
                              void* workspace, size_t workspace_bytes, b200_stream_t stream);

/* Reverse mode of b200_forward with respect to every weight leaf (what
 * jax.vjp through the reference's enzyme_vjp rule, primitives.py:1381-1469,
 * returns for the weight arguments).
 *   dlogits fp32 [batch*seq, vocab]
 *   grads   fp32, packed like the weights (b200_packed_weight_bytes without
 *           transposes, counted in fp32); accumulate != 0 adds into it
 * Use b200_unpack_grads to obtain per-leaf gradients. */
B200_API int32_t b200_backward(B200Plan* plan, const int32_t* tokens, int32_t batch, int32_t seq,
                               const void* packed_w, const float* dlogits, const void* saved,
                               float* grads, int32_t accumulate, void* workspace, size_t workspace_bytes,
                               b200_stream_t stream);
B200_API int32_t b200_packed_grad_bytes(const B200Plan* plan, size_t* bytes);
B200_API int32_t b200_unpack_grads(const B200Plan* plan, const float* grads, float* const* leaves,
                                   b200_stream_t stream);

/* Forward mode (JVP) of b200_forward with respect to every weight leaf: the tangent of the logits for given
 * tangents of the leaves - the `Forward` row of the reference's harness, jax.jvp of the decorated function
 * (test/test_utils.py:689-735), with the forward rules of Implementations/HLODerivatives.td:964-1339 composed per
 * fused block.
 *   packed_dw  the tangents of the 12 leaves, packed with b200_pack_weights exactly like the weights
 *   saved      the activations a b200_forward call with `saved` kept for the same tokens and weights
 *   dlogits    fp32 [batch*seq, vocab], the tangent of the logits
 * One GPU.  The workspace size comes from b200_jvp_workspace_bytes. */
B200_API int32_t b200_jvp_workspace_bytes(const B200Plan* plan, int32_t batch, int32_t seq, size_t* bytes);
B200_API int32_t b200_forward_jvp(B200Plan* plan, const int32_t* tokens, int32_t batch, int32_t seq,
                                  const void* packed_w, const void* packed_dw, const void* saved, float* dlogits,
                                  void* workspace, size_t workspace_bytes, b200_stream_t stream);

/* Forward mode of the reference's own call, forward(x, weights, key_cache, value_cache) -> hidden, with tangents
 * for ALL of its inputs, as the reference's harness passes them (jax.jvp(fn, ins, dins), test/test_utils.py:689-735;
 * `dins` of test/llama.py:316).
 *   dx            fp32 [d]                 packed_dw   the leaf tangents, packed like the weights
 *   d_key_cache   [L, pos, d] of the config dtype (d_value_cache alike); may be NULL when pos == 0
 *   hidden_out    NULL, or fp32 [d] receiving the primal;  d_hidden  fp32 [d], the tangent of the result */
B200_API int32_t b200_token_jvp_workspace_bytes(const B200Plan* plan, int32_t pos, size_t* bytes);
B200_API int32_t b200_token_jvp(B200Plan* plan, const float* x, const void* key_cache, const void* value_cache,
                                int32_t pos, const void* packed_w, const float* dx, const void* packed_dw,
                                const void* d_key_cache, const void* d_value_cache, float* hidden_out,
                                float* d_hidden, void* workspace, size_t workspace_bytes, b200_stream_t stream);

/* Reverse mode of the reference's own call: forward(x, weights, key_cache, value_cache) -> hidden
 * (test/llama.py:35-238), differentiated with respect to ALL of its inputs as the reference's test does
 * (test/llama.py:315-317 `ins`/`dins`, test/test_utils.py:505-514 splatvjp): the residual vector, every weight leaf
 * and both caches.
 *   x            fp32 [d]
 *   key_cache    [L, pos, d] of the config dtype (value_cache alike); may be NULL when pos == 0
 *   packed_w     weights packed with the transposed copies
 *   d_hidden     fp32 [d], the cotangent of the returned hidden state
 *   hidden_out   NULL, or fp32 [d] receiving the primal result (the reference's `revprimal`)
 *   dx           fp32 [d]
 *   grads        fp32, packed like b200_backward's (overwritten).  The hidden state does not depend on wcls
 *                (test/llama.py:236 is commented out) nor on an embedding table: those gradients are exactly
 *                zero, as the reference emits for arguments JAX drops as dead (primitives.py:733-744, :1550-1569).
 *   d_key_cache  fp32 [L, pos, d] (d_value_cache alike)
 * One sequence; the workspace size comes from b200_token_vjp_workspace_bytes. */
B200_API int32_t b200_token_vjp_workspace_bytes(const B200Plan* plan, int32_t pos, size_t* bytes);
/* The primal alone: forward(x, weights, key_cache, value_cache) -> hidden over flat caches [L, pos, d] (the
 * reference's call, test/llama.py:35-238), for a caller that holds the cache as the reference does rather than in
 * pages.  Same workspace size as the VJP. */
B200_API int32_t b200_token_forward(B200Plan* plan, const float* x, const void* key_cache, const void* value_cache,
                                    int32_t pos, const void* packed_w, float* hidden_out, void* workspace,
                                    size_t workspace_bytes, b200_stream_t stream);
/* Buffer sizes for a model on one GPU without a plan and without a device: what a compile-time rewrite needs to type
 * the packed-weight operand, the packed-gradient result and the scratch result of the custom calls it emits (the
 * reference computes its scratch size at lowering time too, primitives.py:712-727).  Any output pointer may be NULL. */
B200_API int32_t b200_static_sizes(const B200LlamaConfig* cfg, int32_t with_transposed, int32_t pos,
                                   size_t* packed_bytes, size_t* grad_bytes, size_t* token_workspace_bytes);
B200_API int32_t b200_token_vjp(B200Plan* plan, const float* x, const void* key_cache, const void* value_cache,
                                int32_t pos, const void* packed_w, const float* d_hidden, float* hidden_out,
                                float* dx, float* grads, float* d_key_cache, float* d_value_cache, void* workspace,
                                size_t workspace_bytes, b200_stream_t stream);

/* Sums `count` floats over the ranks of the communicator in place (the
 * data-parallel gradient exchange). */
B200_API int32_t b200_allreduce_f32(void* comm, float* data, size_t count, b200_stream_t stream);

/* One decode step for `batch` sequences that all hold `pos` cached positions
 * (the reference's single-token `forward`, test/llama.py:35-238, where
 * pos = key_cache.shape[1]).
 *   tokens     int32 [batch], or NULL when x_in is given
 *   x_in       NULL, or fp32 [batch, d] residual vectors (the reference's `x`)
 *   kv_pages   the paged cache: [L, 2, n_pages, H/tp, page_size, head_size] of the
 *              config dtype (head-major pages: the rows of one head are contiguous);
 *              the step appends row `pos` of every sequence
 *   page_table int32 [batch, max_pages]: page index of each sequence's pages
 *   hidden_out NULL, or fp32 [batch, d]: final-normed hidden state (what the
 *              reference returns, test/llama.py:235-238)
 *   logits     NULL, or fp32 [batch, vocab/tp] */
B200_API int32_t b200_decode_step(B200Plan* plan, const int32_t* tokens, const float* x_in, int32_t batch,
                                  int32_t pos, const void* packed_w, void* kv_pages, const int32_t* page_table,
                                  int32_t n_pages, int32_t page_size, int32_t max_pages, float* hidden_out,
                                  float* logits, void* workspace, size_t workspace_bytes, b200_stream_t stream);

/* ---- single kernels (unit-testable pieces of the path) ------------------- */

/* Y[M,N] = A[M,K] * B[N,K]^T with fp32 accumulation; dtype of A and B is
 * in_dtype, of Y out_dtype.  impl: 0 = pick, 1 = tcgen05/TMEM (bf16 only),
 * 2 = FFMA.  ta/tb != 0 read the operand as its transpose ([K,M] / [K,N]). */
B200_API int32_t b200_gemm(const void* A, const void* B, void* Y, int32_t M, int32_t N, int32_t K,
                           int32_t lda, int32_t ldb, int32_t ldy, int32_t ta, int32_t tb, int32_t in_dtype,
                           int32_t out_dtype, int32_t accumulate, int32_t impl, b200_stream_t stream);

/* y = gain * x * rsqrt(mean(x^2) + eps) per row (test/llama.py:6-10). */
B200_API int32_t b200_rmsnorm(const float* x, const float* gain, void* y, float* rinv_or_null, int32_t rows,
                              int32_t dim, float eps, int32_t out_dtype, b200_stream_t stream);

/* Causal attention over [batch, seq] with heads side by side in the rows:
 * q,k,v,o [batch*seq, ld] (test/llama.py:177-209); lse fp32 [batch, H, seq] or NULL. */
B200_API int32_t b200_attention(const void* q, const void* k, const void* v, void* o, float* lse, int32_t batch,
                                int32_t seq, int32_t n_heads, int32_t head_size, int32_t ldq, int32_t ldkv,
                                int32_t ldo, int32_t dtype, int32_t impl, b200_stream_t stream);

/* Reverse mode of b200_attention: given the forward's inputs, output and lse and
 * the cotangent d_o, writes dq, dk, dv (layouts of q, k, v).  delta_scratch is
 * batch*n_heads*seq floats.  The rules are those of
 * Implementations/HLODerivatives.td:1133-1182 (divide, dot_general, exp) composed
 * over test/llama.py:177-209. */
B200_API int32_t b200_attention_backward(const void* q, const void* k, const void* v, const void* o, const float* lse,
                                         const void* d_o, void* dq, void* dk, void* dv, float* delta_scratch,
                                         int32_t batch, int32_t seq, int32_t n_heads, int32_t head_size, int32_t ldq,
                                         int32_t ldkv, int32_t ldo, int32_t dtype, int32_t impl, b200_stream_t stream);

/* Decode attention over the paged cache (test/llama.py:177-209 with a cache of
 * ctx rows): one query row per (sequence, head).
 *   q          [batch, ldq] of `dtype`
 *   kv_pages   one layer of the cache: [2, n_pages, n_heads, page_size, head_size]
 *   page_table int32 [batch, max_pages]
 *   o          [batch, ldo]
 *   scratch    caller-owned, b200_attention_decode_scratch_bytes() bytes: the
 *              per-split partial results between the two kernels */
B200_API int32_t b200_attention_decode_scratch_bytes(int32_t batch, int32_t n_heads, int32_t head_size, int32_t ctx,
                                                     size_t* bytes);
B200_API int32_t b200_attention_decode(const void* q, const void* kv_pages, const int32_t* page_table, void* o,
                                       void* scratch, size_t scratch_bytes, int32_t batch, int32_t ctx,
                                       int32_t n_heads, int32_t head_size, int32_t ldq, int32_t ldo, int32_t n_pages,
                                       int32_t page_size, int32_t max_pages, int32_t dtype, b200_stream_t stream);

/* b200_attention_decode for callers that cannot allocate device memory.  No
 * counterpart in the reference: this entry point exists only in this library.
 * It serves callers that can hand over inputs and outputs but no scratch
 * buffer: a runtime that gives a custom call only its declared operands, a
 * serving loop whose memory pool was fixed at start-up, or code running where
 * cudaMalloc is not permitted.  The per-split partial results live in a 4 MiB
 * array inside the library image (held by every GPU that loads the library
 * until the process exits) instead of a caller buffer; the call itself
 * allocates nothing and frees nothing.
 *  - Limit: batch * n_heads * splits * (head_size + 2) floats must fit in
 *    4 MiB (1,048,576 floats); larger problems return B200_ERR_WORKSPACE and
 *    should use b200_attention_decode with a caller buffer.
 *  - The first call on each device looks up the array's device address (with
 *    that device current).  Make that first call outside any stream capture.
 *  - All calls on a device share the one array.  Two calls whose kernels may
 *    overlap on the GPU (different streams without an ordering between them)
 *    race on it; order them.  Nothing needs clearing between calls: each call
 *    overwrites every slot it later reads. */
B200_API int32_t b200_attention_decode_static(const void* q, const void* kv_pages, const int32_t* page_table,
                                              void* o, int32_t batch, int32_t ctx, int32_t n_heads,
                                              int32_t head_size, int32_t ldq, int32_t ldo, int32_t n_pages,
                                              int32_t page_size, int32_t max_pages, int32_t dtype,
                                              b200_stream_t stream);

/* ---- communicator (NCCL over NVLink) -------------------------------------- */

B200_API int32_t b200_comm_unique_id(void* id128 /* 128 bytes out */);
B200_API int32_t b200_comm_init_rank(const void* id128, int32_t rank, int32_t world, void** comm);
/* Collective over the ranks of the communicator: every rank calls it, after the last work that uses the
 * communicator has been enqueued.  It synchronises the device and then agrees with the peers (a one-element
 * all-reduce) before it frees the exchange buffer and flag words the peers have mapped, so no rank frees memory a
 * slower peer is still reading.  A rank that leaves without calling it must not free that memory some other way
 * while its peers still run kernels of this library. */
B200_API int32_t b200_comm_destroy(void* comm);
/* *enabled = 0 when the tensor-parallel partial sums travel through NCCL, 1 when the ranks exchange them through
 * peer-mapped memory over NVLink with plain loads and stores, 2 when that memory is also bound to a multicast
 * object and the exchange reduces inside the NVLink switch (multimem). */
B200_API int32_t b200_comm_peer_memory(void* comm, int32_t* enabled);

/* b200_comm_init_rank with own_peer_memory = 0 creates the communicator without its own exchange buffers, for a
 * caller that brings them with b200_comm_attach_memory; b200_comm_setup_peer_memory (collective) creates the
 * library's own (CUDA IPC) afterwards, e.g. when the attach was refused. */
B200_API int32_t b200_comm_init_rank_ex(const void* id128, int32_t rank, int32_t world, int32_t own_peer_memory,
                                        void** comm);
B200_API int32_t b200_comm_setup_peer_memory(void* comm);

/* Hands the communicator exchange memory the CALLER owns: `bytes` (a multiple of 256, at least 8 MiB + 4 KiB) of
 * device memory on every rank, of which peer_ptrs[r] is rank r's block as mapped into this process
 * (peer_ptrs[rank] is this rank's own), and multicast_ptr the address of a multicast mapping of the same blocks
 * (cuMulticastCreate / cuMulticastBindMem; NULL when there is none).  Collective: every rank calls it with its own
 * view, before the communicator is used by a plan.  The last 4 KiB of the block hold the flag words and are cleared
 * here.  The library never frees this memory; the caller keeps it alive until after b200_comm_destroy.  Returns
 * B200_ERR_UNSUPPORTED on every rank when some rank could not attach (the communicator then still has no exchange
 * memory).  With a multicast address the tensor-parallel exchange of the prefill sums inside the NVLink switch
 * (multimem.ld_reduce / multimem.st): 1/world of the bytes cross each link.
 * The reference has no counterpart (it has no multi-GPU runtime); symmetric-memory allocators (for example
 * torch.distributed's, which the Python host of this library uses) provide such blocks. */
B200_API int32_t b200_comm_attach_memory(void* comm, size_t bytes, const void* const* peer_ptrs, void* multicast_ptr);

/* The exchange of the tensor-parallel prefill as a single kernel (unit-testable piece of the path).  Every rank owns
 * rows_total / world consecutive rows of the fp32 residual stream (x_own, [rows_total / world, dim]).
 * b200_tp_exchange_buffers gives the two regions of this rank's exchange memory: `part`, where the rank leaves its
 * partial product [rows_total, dim] of `dtype` (what the row-parallel Wo / W2 projection writes), and `gathered`,
 * where the normed rows of ALL ranks arrive.  b200_tp_reduce_norm (collective, same arguments on every rank) then,
 * for this rank's rows: x_own += sum over ranks of part (skipped when reduce == 0), and gain * x_own * rsqrt(mean
 * x_own^2 + eps) goes to `gathered` on every rank; when the call's kernel has completed, this rank's `gathered`
 * holds all rows_total rows.  It stands for test/llama.py:211-219 (`x += wo @ ...` followed by rmsnorm) under the
 * Megatron split, where the reference has no multi-GPU code. */
B200_API int32_t b200_tp_exchange_buffers(void* comm, size_t bytes_each, void** part, void** gathered);
B200_API int32_t b200_tp_reduce_norm(void* comm, int32_t rows_total, int32_t dim, int32_t dtype, int32_t reduce,
                                     float* x_own, const float* gain, float eps, b200_stream_t stream);

/* ---- XLA FFI registration -------------------------------------------------- */

/* Custom-call targets of the typed FFI (api_version 4), the counterpart of registerEnzymeJaXXLAFFI()
 * (src/enzyme_ad/jax/xla_ffi/register.cc:21-27, handlers bound as in xla_ffi/cuda/blas.cc:257-314):
 *   enzymejax_b200_llama_pack         leaves (12 buffers, B200Leaf order) -> packed weights
 *   enzymejax_b200_llama_fwd          tokens, packed -> logits, workspace
 *   enzymejax_b200_llama_fwd_saved    tokens, packed -> logits, saved activations, workspace
 *   enzymejax_b200_llama_bwd          tokens, packed, dlogits, saved -> packed gradients, workspace
 *   enzymejax_b200_llama_unpack_grads packed gradients -> 12 gradient leaves
 *   enzymejax_b200_llama_decode_step  tokens, packed, kv pages (aliased in place), page table -> logits, workspace
 *   enzymejax_b200_llama_token_fwd    x, packed, key_cache, value_cache -> hidden, workspace   (the reference's call)
 *   enzymejax_b200_llama_token_vjp    x, packed, key_cache, value_cache, d_hidden -> hidden, dx, packed gradients,
 *                                     d_key_cache, d_value_cache, workspace
 * The handlers exist only in a library built where the XLA FFI headers (xla/ffi/api/ffi.h, shipped inside jaxlib)
 * are on the include path; b200_ffi_available() says whether this build has them.
 *
 * b200_ffi_handler(name) returns the handler's address (an XLA_FFI_Handler*), or NULL for an unknown name or a
 * build without the headers.  A Python host wraps it in a PyCapsule named "xla._CUSTOM_CALL_TARGET" and hands it to
 * jax.ffi.register_ffi_target(name, capsule, platform="CUDA") - the route the reference takes for its legacy
 * targets (primitives.py:32-37, capsule made in enzyme_call.cc:527-530).
 *
 * registerEnzymeJaXB200FFI() registers all targets with the XLA instance linked into the calling process through
 * XLA_FFI_REGISTER_HANDLER; idempotent; returns B200_ERR_UNSUPPORTED in a build without the headers. */
B200_API int32_t b200_ffi_available(void);
B200_API void* b200_ffi_handler(const char* target_name);
B200_API int32_t registerEnzymeJaXB200FFI(void);

#ifdef __cplusplus
}
#endif
#endif /* B200_LLAMA_H_ */

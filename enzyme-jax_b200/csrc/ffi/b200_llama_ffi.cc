// XLA typed-FFI (api_version 4) custom-call targets of the llama path.
//
// Each handler unpacks its attributes and buffers and calls the C ABI of
// include/b200_llama.h on the stream XLA hands it; it allocates nothing (scratch
// arrives as an extra i8 result, the way the reference's legacy path appends an
// i8[tmpBuf] result, primitives.py:712-727), never synchronises (gpu.cc:122-125,153)
// and turns a non-zero status into ffi::Error with the library's message (as
// xla_ffi/cuda/blas.cc:80-115 does for cuBLAS failures).  Binding and definition
// follow the reference's idiom, xla_ffi/cuda/blas.cc:257-314; one-time
// registration follows xla_ffi/register.cc:21-27.
//
// The handlers need the XLA FFI headers that jaxlib ships (xla/ffi/api/ffi.h).
// Without them this file still compiles: the three exported functions then
// report that the build has no handlers.
#include <dlfcn.h>
#include <string.h>

#include <mutex>

#include "../../../include/b200_llama.h"

#if defined(__has_include)
#if __has_include("xla/ffi/api/ffi.h")
#define B200_HAVE_XLA_FFI 1
#endif
#endif

#ifdef B200_HAVE_XLA_FFI

#include <cuda_runtime_api.h>

#include <string>

#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error status_to_error(int32_t st) {
  if (st == B200_OK) return ffi::Error::Success();
  const std::string msg = std::string("b200_llama: ") + b200_last_error();
  switch (st) {
    case B200_ERR_INVALID_ARG:
    case B200_ERR_BAD_SHAPE:
    case B200_ERR_BAD_DTYPE:
    case B200_ERR_MISALIGNED:
    case B200_ERR_WORKSPACE:
      return ffi::Error::InvalidArgument(msg);
    case B200_ERR_UNSUPPORTED:
    case B200_ERR_ARCH:
      return ffi::Error(ffi::ErrorCode::kUnimplemented, msg);
    default:
      return ffi::Error::Internal(msg);
  }
}

#define B200_FFI_TRY(expr)                                  \
  do {                                                      \
    const int32_t _st = (expr);                             \
    if (_st != B200_OK) return status_to_error(_st);        \
  } while (0)

// The model attributes every target carries (backend_config of the custom call).
struct ModelAttrs {
  int32_t dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len, dtype;
  float rope_theta, rms_eps;
};

ffi::Error plan_for(const ModelAttrs& m, B200Plan** plan) {
  B200LlamaConfig cfg;
  cfg.dim = m.dim; cfg.hidden_dim = m.hidden_dim; cfg.n_layers = m.n_layers; cfg.n_heads = m.n_heads;
  cfg.n_kv_heads = m.n_kv_heads; cfg.vocab_size = m.vocab_size; cfg.seq_len = m.seq_len; cfg.dtype = m.dtype;
  cfg.rope_theta = m.rope_theta; cfg.rms_eps = m.rms_eps;
  // one process per GPU under jit: tensor parallelism is set up by the Python host (b200_comm_init_rank), the
  // jitted single-device call is tp_size 1
  return status_to_error(b200_plan_cached(&cfg, 0, 1, nullptr, plan));
}

int32_t leaf_dtype_of(ffi::DataType t) {
  if (t == ffi::DataType::F32) return B200_F32;
  if (t == ffi::DataType::BF16) return B200_BF16;
  return -1;
}

#define B200_MODEL_ATTRS                                                                                          \
  int32_t dim, int32_t hidden_dim, int32_t n_layers, int32_t n_heads, int32_t n_kv_heads, int32_t vocab_size,    \
      int32_t seq_len, int32_t dtype, float rope_theta, float rms_eps
#define B200_MODEL_ATTRS_PACK \
  ModelAttrs { dim, hidden_dim, n_layers, n_heads, n_kv_heads, vocab_size, seq_len, dtype, rope_theta, rms_eps }
#define B200_BIND_MODEL_ATTRS(b)                                                                                  \
  b.Attr<int32_t>("dim").Attr<int32_t>("hidden_dim").Attr<int32_t>("n_layers").Attr<int32_t>("n_heads")           \
      .Attr<int32_t>("n_kv_heads").Attr<int32_t>("vocab_size").Attr<int32_t>("seq_len").Attr<int32_t>("dtype")    \
      .Attr<float>("rope_theta").Attr<float>("rms_eps")

// ---- pack: 12 leaves (B200Leaf order) -> packed weights ------------------------------------
ffi::Error PackImpl(cudaStream_t stream, B200_MODEL_ATTRS, bool with_transposed, ffi::RemainingArgs leaves,
                    ffi::Result<ffi::AnyBuffer> packed) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  if (leaves.size() != B200_NUM_LEAVES) return ffi::Error::InvalidArgument("b200_llama pack: expected 12 weight leaves");
  const void* ptrs[B200_NUM_LEAVES];
  int32_t ldt = -1;
  for (size_t i = 0; i < B200_NUM_LEAVES; ++i) {
    auto buf = leaves.get<ffi::AnyBuffer>(i);
    if (!buf.has_value()) return buf.error();
    ptrs[i] = buf->untyped_data();
    const int32_t t = leaf_dtype_of(buf->element_type());
    if (t < 0 || (ldt >= 0 && t != ldt)) return ffi::Error::InvalidArgument("b200_llama pack: leaves must all be f32 or all bf16");
    ldt = t;
  }
  size_t need = 0;
  B200_FFI_TRY(b200_packed_weight_bytes(plan, with_transposed ? 1 : 0, &need));
  if (packed->size_bytes() < need) return ffi::Error::InvalidArgument("b200_llama pack: packed buffer too small");
  B200_FFI_TRY(b200_pack_weights(plan, ptrs, ldt, with_transposed ? 1 : 0, packed->untyped_data(), stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaPack, PackImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Attr<bool>("with_transposed")
                                  .RemainingArgs()
                                  .Ret<ffi::AnyBuffer>());

// ---- forward: tokens [B,S] s32, packed -> logits [B,S,V] f32, workspace i8 ---------------------
ffi::Error FwdImpl(cudaStream_t stream, B200_MODEL_ATTRS, ffi::AnyBuffer tokens, ffi::AnyBuffer packed,
                   ffi::Result<ffi::AnyBuffer> logits, ffi::Result<ffi::AnyBuffer> workspace) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  const auto dims = tokens.dimensions();
  if (dims.size() != 2 || tokens.element_type() != ffi::DataType::S32)
    return ffi::Error::InvalidArgument("b200_llama fwd: tokens must be s32[batch, seq]");
  B200_FFI_TRY(b200_forward(plan, static_cast<const int32_t*>(tokens.untyped_data()), (int32_t)dims[0],
                            (int32_t)dims[1], packed.untyped_data(), static_cast<float*>(logits->untyped_data()),
                            nullptr, nullptr, workspace->untyped_data(), workspace->size_bytes(), stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaFwd, FwdImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());

// ---- forward keeping activations (the primal half of jax.vjp) -------------------------------------
ffi::Error FwdSavedImpl(cudaStream_t stream, B200_MODEL_ATTRS, ffi::AnyBuffer tokens, ffi::AnyBuffer packed,
                        ffi::Result<ffi::AnyBuffer> logits, ffi::Result<ffi::AnyBuffer> saved,
                        ffi::Result<ffi::AnyBuffer> workspace) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  const auto dims = tokens.dimensions();
  if (dims.size() != 2 || tokens.element_type() != ffi::DataType::S32)
    return ffi::Error::InvalidArgument("b200_llama fwd_saved: tokens must be s32[batch, seq]");
  size_t need = 0;
  B200_FFI_TRY(b200_saved_bytes(plan, (int32_t)dims[0], (int32_t)dims[1], &need));
  if (saved->size_bytes() < need) return ffi::Error::InvalidArgument("b200_llama fwd_saved: saved buffer too small");
  B200_FFI_TRY(b200_forward(plan, static_cast<const int32_t*>(tokens.untyped_data()), (int32_t)dims[0],
                            (int32_t)dims[1], packed.untyped_data(), static_cast<float*>(logits->untyped_data()),
                            saved->untyped_data(), nullptr, workspace->untyped_data(), workspace->size_bytes(),
                            stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaFwdSaved, FwdSavedImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());

// ---- backward: tokens, packed (with transposes), dlogits, saved -> packed gradients, workspace --------
ffi::Error BwdImpl(cudaStream_t stream, B200_MODEL_ATTRS, ffi::AnyBuffer tokens, ffi::AnyBuffer packed,
                   ffi::AnyBuffer dlogits, ffi::AnyBuffer saved, ffi::Result<ffi::AnyBuffer> grads,
                   ffi::Result<ffi::AnyBuffer> workspace) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  const auto dims = tokens.dimensions();
  if (dims.size() != 2 || tokens.element_type() != ffi::DataType::S32)
    return ffi::Error::InvalidArgument("b200_llama bwd: tokens must be s32[batch, seq]");
  if (dlogits.element_type() != ffi::DataType::F32)
    return ffi::Error::InvalidArgument("b200_llama bwd: the cotangent of the logits must be f32");
  size_t need = 0;
  B200_FFI_TRY(b200_packed_grad_bytes(plan, &need));
  if (grads->size_bytes() < need) return ffi::Error::InvalidArgument("b200_llama bwd: gradient buffer too small");
  B200_FFI_TRY(b200_backward(plan, static_cast<const int32_t*>(tokens.untyped_data()), (int32_t)dims[0],
                             (int32_t)dims[1], packed.untyped_data(), static_cast<const float*>(dlogits.untyped_data()),
                             saved.untyped_data(), static_cast<float*>(grads->untyped_data()), /*accumulate=*/0,
                             workspace->untyped_data(), workspace->size_bytes(), stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaBwd, BwdImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());

// ---- packed gradients -> 12 gradient leaves (f32, B200Leaf order) ----------------------------------
ffi::Error UnpackGradsImpl(cudaStream_t stream, B200_MODEL_ATTRS, ffi::AnyBuffer grads, ffi::RemainingRets leaves) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  if (leaves.size() != B200_NUM_LEAVES) return ffi::Error::InvalidArgument("b200_llama unpack_grads: expected 12 results");
  float* ptrs[B200_NUM_LEAVES];
  for (size_t i = 0; i < B200_NUM_LEAVES; ++i) {
    auto buf = leaves.get<ffi::AnyBuffer>(i);
    if (!buf.has_value()) return buf.error();
    if ((*buf)->element_type() != ffi::DataType::F32)
      return ffi::Error::InvalidArgument("b200_llama unpack_grads: gradient leaves are f32");
    ptrs[i] = static_cast<float*>((*buf)->untyped_data());
  }
  B200_FFI_TRY(b200_unpack_grads(plan, static_cast<const float*>(grads.untyped_data()), ptrs, stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaUnpackGrads, UnpackGradsImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Arg<ffi::AnyBuffer>()
                                  .RemainingRets());

// ---- decode step: the cache operand is aliased to the cache result (output_operand_aliases) ----------
ffi::Error DecodeImpl(cudaStream_t stream, B200_MODEL_ATTRS, int32_t pos, int32_t page_size, ffi::AnyBuffer tokens,
                      ffi::AnyBuffer packed, ffi::AnyBuffer kv_in, ffi::AnyBuffer page_table,
                      ffi::Result<ffi::AnyBuffer> logits, ffi::Result<ffi::AnyBuffer> kv_out,
                      ffi::Result<ffi::AnyBuffer> workspace) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  const auto tdims = tokens.dimensions();
  const auto pdims = page_table.dimensions();
  const auto kdims = kv_in.dimensions();  // [L, 2, n_pages, H, page_size, head_size]
  if (tdims.size() != 1 || pdims.size() != 2 || kdims.size() != 6 || tokens.element_type() != ffi::DataType::S32 ||
      page_table.element_type() != ffi::DataType::S32)
    return ffi::Error::InvalidArgument("b200_llama decode_step: tokens s32[batch], page_table s32[batch, max_pages], "
                                       "cache [L, 2, n_pages, H, page_size, head_size]");
  // in-place update is expressed by the alias; if XLA still hands two buffers, copy first (as blas.cc:218-226 does)
  if (kv_in.untyped_data() != kv_out->untyped_data()) {
    if (cudaMemcpyAsync(kv_out->untyped_data(), kv_in.untyped_data(), kv_in.size_bytes(), cudaMemcpyDeviceToDevice,
                        stream) != cudaSuccess)
      return ffi::Error::Internal("b200_llama decode_step: copying the cache failed");
  }
  B200_FFI_TRY(b200_decode_step(plan, static_cast<const int32_t*>(tokens.untyped_data()), nullptr, (int32_t)tdims[0], pos,
                                packed.untyped_data(), kv_out->untyped_data(),
                                static_cast<const int32_t*>(page_table.untyped_data()), (int32_t)kdims[2], page_size,
                                (int32_t)pdims[1], nullptr, static_cast<float*>(logits->untyped_data()),
                                workspace->untyped_data(), workspace->size_bytes(), stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaDecodeStep, DecodeImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Attr<int32_t>("pos")
                                  .Attr<int32_t>("page_size")
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());

// The FFI api table of the XLA linked into this process, when it exports one (looked up by name so that this
// library does not need XLA at link time).
const XLA_FFI_Api* b200_xla_api() {
  using GetApiFn = const XLA_FFI_Api* (*)();
  static const XLA_FFI_Api* api = [] {
    GetApiFn fn = reinterpret_cast<GetApiFn>(dlsym(RTLD_DEFAULT, "GetXlaFfiApi"));
    if (!fn) fn = reinterpret_cast<GetApiFn>(dlsym(RTLD_DEFAULT, "_ZN3xla3ffi12GetXlaFfiApiEv"));  // xla::ffi::GetXlaFfiApi()
    return fn ? fn() : nullptr;
  }();
  return api;
}

// ---- the reference's own call over flat caches [L, pos, d] ---------------------------------------------
ffi::Error TokenFwdImpl(cudaStream_t stream, B200_MODEL_ATTRS, ffi::AnyBuffer x, ffi::AnyBuffer packed,
                        ffi::AnyBuffer key_cache, ffi::AnyBuffer value_cache, ffi::Result<ffi::AnyBuffer> hidden,
                        ffi::Result<ffi::AnyBuffer> workspace) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  const auto kd = key_cache.dimensions();
  if (kd.size() != 3 || x.element_type() != ffi::DataType::F32)
    return ffi::Error::InvalidArgument("b200_llama token_fwd: x f32[dim], caches [n_layers, pos, dim]");
  B200_FFI_TRY(b200_token_forward(plan, static_cast<const float*>(x.untyped_data()), key_cache.untyped_data(),
                                  value_cache.untyped_data(), (int32_t)kd[1], packed.untyped_data(),
                                  static_cast<float*>(hidden->untyped_data()), workspace->untyped_data(),
                                  workspace->size_bytes(), stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaTokenFwd, TokenFwdImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());

ffi::Error TokenVjpImpl(cudaStream_t stream, B200_MODEL_ATTRS, ffi::AnyBuffer x, ffi::AnyBuffer packed,
                        ffi::AnyBuffer key_cache, ffi::AnyBuffer value_cache, ffi::AnyBuffer d_hidden,
                        ffi::Result<ffi::AnyBuffer> hidden, ffi::Result<ffi::AnyBuffer> dx,
                        ffi::Result<ffi::AnyBuffer> grads, ffi::Result<ffi::AnyBuffer> d_key_cache,
                        ffi::Result<ffi::AnyBuffer> d_value_cache, ffi::Result<ffi::AnyBuffer> workspace) {
  B200Plan* plan = nullptr;
  if (ffi::Error e = plan_for(B200_MODEL_ATTRS_PACK, &plan); e.failure()) return e;
  const auto kd = key_cache.dimensions();
  if (kd.size() != 3 || x.element_type() != ffi::DataType::F32 || d_hidden.element_type() != ffi::DataType::F32)
    return ffi::Error::InvalidArgument("b200_llama token_vjp: x and d_hidden f32[dim], caches [n_layers, pos, dim]");
  B200_FFI_TRY(b200_token_vjp(plan, static_cast<const float*>(x.untyped_data()), key_cache.untyped_data(),
                              value_cache.untyped_data(), (int32_t)kd[1], packed.untyped_data(),
                              static_cast<const float*>(d_hidden.untyped_data()),
                              static_cast<float*>(hidden->untyped_data()), static_cast<float*>(dx->untyped_data()),
                              static_cast<float*>(grads->untyped_data()),
                              static_cast<float*>(d_key_cache->untyped_data()),
                              static_cast<float*>(d_value_cache->untyped_data()), workspace->untyped_data(),
                              workspace->size_bytes(), stream));
  return ffi::Error::Success();
}
XLA_FFI_DEFINE_HANDLER_SYMBOL(B200LlamaTokenVjp, TokenVjpImpl,
                              B200_BIND_MODEL_ATTRS(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>())
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>());

struct Target { const char* name; XLA_FFI_Handler* handler; };
const Target kTargets[] = {
    {"enzymejax_b200_llama_pack", B200LlamaPack},
    {"enzymejax_b200_llama_fwd", B200LlamaFwd},
    {"enzymejax_b200_llama_fwd_saved", B200LlamaFwdSaved},
    {"enzymejax_b200_llama_bwd", B200LlamaBwd},
    {"enzymejax_b200_llama_unpack_grads", B200LlamaUnpackGrads},
    {"enzymejax_b200_llama_decode_step", B200LlamaDecodeStep},
    {"enzymejax_b200_llama_token_fwd", B200LlamaTokenFwd},
    {"enzymejax_b200_llama_token_vjp", B200LlamaTokenVjp},
};

}  // namespace

extern "C" {

int32_t b200_ffi_available(void) { return 1; }

void* b200_ffi_handler(const char* name) {
  if (!name) return nullptr;
  for (const Target& t : kTargets)
    if (strcmp(t.name, name) == 0) return reinterpret_cast<void*>(t.handler);
  return nullptr;
}

// In a process whose XLA exports its FFI api table (the reference's own extension links XLA, register.cc:21-27), the
// targets are registered directly; elsewhere the host registers the handler addresses through
// jax.ffi.register_ffi_target.
int32_t registerEnzymeJaXB200FFI(void) {
  static std::once_flag once;
  static int32_t result = B200_ERR_UNSUPPORTED;
  std::call_once(once, [] {
    if (!b200_xla_api()) return;
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_pack", "CUDA", B200LlamaPack);
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_fwd", "CUDA", B200LlamaFwd);
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_fwd_saved", "CUDA", B200LlamaFwdSaved);
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_bwd", "CUDA", B200LlamaBwd);
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_unpack_grads", "CUDA", B200LlamaUnpackGrads);
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_decode_step", "CUDA", B200LlamaDecodeStep);
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_token_fwd", "CUDA", B200LlamaTokenFwd);
    XLA_FFI_REGISTER_HANDLER(b200_xla_api(), "enzymejax_b200_llama_token_vjp", "CUDA", B200LlamaTokenVjp);
    result = B200_OK;
  });
  return result;
}

}  // extern "C"

#else  // no XLA FFI headers at build time

extern "C" {

int32_t b200_ffi_available(void) { return 0; }
void* b200_ffi_handler(const char*) { return nullptr; }
int32_t registerEnzymeJaXB200FFI(void) { return B200_ERR_UNSUPPORTED; }

}  // extern "C"

#endif

"""The reference's Python surface for the llama path, backed by the B200 library.

Mirrors the names of the reference's ``enzyme_ad.jax`` package
(``src/enzyme_ad/jax/__init__.py:1-12``): ``enzyme_jax_ir`` keeps its signature
(``primitives.py:1528``), the pipeline classes keep their methods
(``primitives.py:56-115``).  JAX is not installed where this runs, so the
decorated function takes and returns torch CUDA tensors; under JAX the same
routing sits behind ``jax.ffi.ffi_call`` and ``jax.custom_vjp``.

Only the llama path is implemented.  ``B200Pipeline(config)`` is the caller's
declaration that the decorated function IS the llama forward of that config; the
decorator then holds the call to it: the function must accept the arguments it
is called with (``inspect.signature``), the weight dict must have exactly the
reference's leaves with the shapes the config implies (test/llama.py:270-282),
and the other arguments the shapes of test/llama.py:288-301.  Anything else
raises instead of silently computing llama.  Two call shapes exist:

* ``fn(x, weights, key_cache, value_cache)`` -- the reference's own call
  (``test/llama.py:35``, ``:288-292``): one fp32 residual vector ``[dim]`` and
  caches ``[n_layers, pos, kv_dim]``; returns the final-normed hidden ``[dim]``.
* ``fn(tokens, weights)`` with int tokens ``[batch, seq]`` -- the full causal
  forward with embedding and logits; returns fp32 logits ``[batch, seq, vocab]``.

Everything else of the reference's surface (MLIR pipelines, ``cpp_call``,
``hlo_call``, ``export``) raises ``NotImplementedError``: there is no fallback.
"""
from __future__ import annotations

import functools
import inspect
from typing import Callable, Dict, Optional, Tuple

import torch

import b200_llama as _B

WEIGHT_KEYS = ("rms_att_weight", "rms_ffn_weight", "rms_final_weight", "w1", "w2", "w3", "wcls", "wk", "wo", "wq", "wv")


class PipelineConfig:
    def xla_runtime(self):
        raise NotImplementedError()

    def pass_pipeline(self):
        raise NotImplementedError()

    def mlir_ad(self):
        raise NotImplementedError()

    def stablehlo_inject(self):
        raise NotImplementedError()

    def ad_level(self):
        raise NotImplementedError()

    def export_llvm(self):
        raise NotImplementedError()


class XLAPipeline:
    """Reference: primitives.py:81-98."""

    def __init__(self, name=None):
        self.exportname = name

    def xla_runtime(self):
        return False

    def pass_pipeline(self):
        return ""

    def mlir_ad(self):
        return False

    def stablehlo_inject(self):
        return False

    def export_llvm(self):
        return self.exportname


class JaXPipeline:
    """Reference: primitives.py:101-115.  Holds a pass string; running MLIR
    passes is not part of this build."""

    def __init__(self, passes=""):
        self.passes = passes

    def pass_pipeline(self):
        return self.passes

    def mlir_ad(self):
        return True

    def stablehlo_inject(self):
        return True

    def ad_level(self):
        return self.passes.count("enzyme-wrap")


class B200Pipeline(JaXPipeline):
    """Routes the decorated llama function to the sm_100a kernel library.

    ``config`` is the reference's config dict (test/llama.py:246-254);
    ``dtype`` the storage type of weights and activations."""

    def __init__(self, config: Dict[str, int], dtype: torch.dtype = torch.float32, tp_rank: int = 0, tp_size: int = 1,
                 comm=None):
        super().__init__("")
        self.config = dict(config)
        self.dtype = dtype
        self.tp_rank, self.tp_size, self.comm = tp_rank, tp_size, comm

    def stablehlo_inject(self):
        return False


def _unsupported(name):
    def fn(*a, **k):
        raise NotImplementedError(
            f"enzyme_ad.jax.{name} belongs to the reference's MLIR/clang compiler, which this B200 build does not "
            "contain; only the llama forward / VJP path behind enzyme_jax_ir(pipeline_options=B200Pipeline(...)) exists")
    fn.__name__ = name
    return fn


cpp_call = _unsupported("cpp_call")
hlo_call = _unsupported("hlo_call")
ffi_call = _unsupported("ffi_call")
optimize_module = _unsupported("optimize_module")
export = _unsupported("export")
optimization_passes = _unsupported("optimization_passes")
full_optimization_pass_pipeline = _unsupported("full_optimization_pass_pipeline")


def reference_weight_shapes(config: Dict[str, int]) -> Dict[str, Tuple[int, ...]]:
    """Leaf names and shapes of the reference's weight dict (test/llama.py:270-282; the projections are used as
    [out, in], :149-157, and kv_dim == dim because n_kv_heads == n_heads)."""
    L, d, h, V = config["n_layers"], config["dim"], config["hidden_dim"], config["vocab_size"]
    return {"rms_att_weight": (L, d), "rms_ffn_weight": (L, d), "rms_final_weight": (d,), "w1": (L, h, d),
            "w2": (L, d, h), "w3": (L, h, d), "wcls": (V, d), "wk": (L, d, d), "wo": (L, d, d), "wq": (L, d, d),
            "wv": (L, d, d)}


def check_weights(weights, config: Dict[str, int], need_embedding: bool) -> None:
    """Raises unless ``weights`` is the reference's weight dict for ``config`` (plus ``token_embedding_table``
    [vocab, dim] for the token call shape)."""
    if not isinstance(weights, dict):
        raise TypeError("weights must be the reference's dict of weight leaves")
    want = reference_weight_shapes(config)
    if need_embedding:
        want["token_embedding_table"] = (config["vocab_size"], config["dim"])
    extra = sorted(set(weights) - set(want) - {"token_embedding_table"})
    missing = sorted(set(want) - set(weights))
    if extra or missing:
        raise ValueError(f"not the llama weight dict: missing leaves {missing}, unknown leaves {extra}")
    for name, shape in want.items():
        if tuple(weights[name].shape) != shape:
            raise ValueError(f"leaf {name} has shape {tuple(weights[name].shape)}, the config implies {shape}")


def _bind_or_raise(func: Callable, args) -> None:
    """The decorated function must accept the call: the decorator replaces its body, not its signature."""
    try:
        sig = inspect.signature(func)
    except (TypeError, ValueError):
        return  # builtins and the like carry no signature
    try:
        sig.bind(*args)
    except TypeError as exc:
        raise TypeError(f"{getattr(func, '__name__', 'function')} cannot be called with {len(args)} arguments: {exc}") from exc


class _LlamaRoute:
    """One plan per (device, weight identity): packs the weights on first use."""

    def __init__(self, pipe: B200Pipeline):
        self.pipe = pipe
        self.plan: Optional[_B.Plan] = None
        self.weights_key = None
        self.with_t = False

    def _ensure(self, weights: Dict[str, torch.Tensor], with_t: bool):
        key = tuple((k, weights[k].data_ptr(), weights[k]._version) for k in sorted(weights))
        if self.plan is None:
            self.plan = _B.Plan(self.pipe.config, self.pipe.dtype, tp_rank=self.pipe.tp_rank, tp_size=self.pipe.tp_size,
                                comm=self.pipe.comm)
        if key != self.weights_key or (with_t and not self.with_t):
            cfg = self.pipe.config
            full = dict(weights)
            if "token_embedding_table" not in full:
                # the reference's test has no embedding leaf (test/llama.py:109-113 is commented out)
                full["token_embedding_table"] = torch.zeros(cfg["vocab_size"], cfg["dim"], dtype=self.pipe.dtype,
                                                            device=self.plan.device)
            full = {k: v.to(device=self.plan.device, dtype=self.pipe.dtype).contiguous() for k, v in full.items()}
            self.plan.pack_weights(full, with_transposed=with_t)
            self.weights_key, self.with_t = key, with_t
        return self.plan

    # fn(x, weights, key_cache, value_cache) -> hidden [dim]
    def check_token_call(self, x, weights, key_cache, value_cache):
        cfg = self.pipe.config
        check_weights(weights, cfg, need_embedding=False)
        L, d = cfg["n_layers"], cfg["dim"]
        if tuple(x.shape) != (d,) or not x.dtype.is_floating_point:
            raise ValueError(f"x must be a floating-point vector [{d}] (test/llama.py:288), got {tuple(x.shape)} {x.dtype}")
        for name, c in (("key_cache", key_cache), ("value_cache", value_cache)):
            if c.dim() != 3 or c.shape[0] != L or c.shape[2] != d:
                raise ValueError(f"{name} must be [{L}, pos, {d}] (test/llama.py:299-301), got {tuple(c.shape)}")
        if key_cache.shape != value_cache.shape:
            raise ValueError("key_cache and value_cache must have the same shape")
        if key_cache.shape[1] >= cfg["seq_len"]:
            raise ValueError(f"a cache of {key_cache.shape[1]} rows leaves no position below seq_len={cfg['seq_len']}")

    def decode_hidden(self, x, weights, key_cache, value_cache):
        self.check_token_call(x, weights, key_cache, value_cache)
        plan = self._ensure(weights, False)
        cfg = self.pipe.config
        L, pos = key_cache.shape[0], key_cache.shape[1]
        page = max(16, 1 << (pos).bit_length())
        kv = plan.new_kv_pages(1, page)
        if pos:
            H = cfg["n_heads"]
            hs = cfg["dim"] // H
            # [L, pos, kv_dim] -> head-major page [L, H, pos, hs]
            kv[:, 0, 0, :, :pos] = key_cache.to(plan.device, self.pipe.dtype).view(L, pos, H, hs).permute(0, 2, 1, 3)
            kv[:, 1, 0, :, :pos] = value_cache.to(plan.device, self.pipe.dtype).view(L, pos, H, hs).permute(0, 2, 1, 3)
        table = torch.zeros(1, 1, dtype=torch.int32, device=plan.device)
        xin = x.to(plan.device, torch.float32).reshape(1, cfg["dim"]).contiguous()
        hidden, _ = plan.decode_step(pos, kv, table, x=xin, want_hidden=True, want_logits=False)
        return hidden[0]

    # fn(tokens, weights) -> logits
    def check_sequence_call(self, tokens, weights):
        cfg = self.pipe.config
        check_weights(weights, cfg, need_embedding=True)
        if tokens.dim() != 2 or tokens.dtype.is_floating_point:
            raise ValueError(f"tokens must be integers [batch, seq], got {tuple(tokens.shape)} {tokens.dtype}")
        if tokens.shape[1] > cfg["seq_len"]:
            raise ValueError(f"{tokens.shape[1]} positions exceed seq_len={cfg['seq_len']}")

    def forward_logits(self, tokens, weights, saved=None):
        self.check_sequence_call(tokens, weights)
        plan = self._ensure(weights, saved is not None)
        return plan.forward(tokens.to(plan.device, torch.int32).contiguous(), saved=saved)


def enzyme_jax_ir(argv=(), pipeline_options=None, jit_options=None, inner_jit=True):
    """Decorator with the reference's signature (primitives.py:1528).  With a
    ``B200Pipeline`` the wrapped llama function runs on the sm_100a library; any
    other pipeline object is rejected (no MLIR here)."""

    def decorator(func: Callable):
        if not isinstance(pipeline_options, B200Pipeline):
            raise NotImplementedError("this build only executes functions given pipeline_options=B200Pipeline(config)")
        route = _LlamaRoute(pipeline_options)

        @functools.wraps(func)
        def wrapped(*args, **kwargs):
            if kwargs:
                raise NotImplementedError("keyword arguments are not part of the llama call shapes")
            _bind_or_raise(func, args)
            if len(args) == 4 and isinstance(args[1], dict):
                return route.decode_hidden(*args)
            if len(args) == 2 and isinstance(args[1], dict):
                return route.forward_logits(*args)
            raise NotImplementedError(
                "unrecognised call: expected (x, weights, key_cache, value_cache) or (tokens, weights)")

        wrapped._b200_route = route
        return wrapped

    return decorator


def vjp(fn: Callable, *primals):
    """``jax.vjp``-shaped helper for a decorated llama function: ``out, pullback = vjp(fn, *primals)``;
    ``pullback(cotangent)`` returns one cotangent per primal, as ``jax.vjp`` does through the reference's
    ``enzyme_vjp`` rule (primitives.py:1381-1469).

    * ``vjp(fn, x, weights, key_cache, value_cache)`` -- the reference's differentiated call (test/llama.py:315-317,
      test/test_utils.py:505-514): ``out`` is the hidden state ``[dim]``, the pullback maps ``d_hidden`` to
      ``(dx, dweights, d_key_cache, d_value_cache)``.  ``dweights`` has the keys of ``weights``; ``wcls`` comes out
      identically zero -- the function does not use it, and the reference likewise emits zeros for arguments JAX
      drops as dead (primitives.py:733-744, :1550-1569).
    * ``vjp(fn, tokens, weights)`` -- the sequence form: ``out`` is the logits, the pullback maps ``dlogits`` to
      ``(None, dweights)`` (integer tokens carry no cotangent)."""
    route: _LlamaRoute = getattr(fn, "_b200_route", None)
    if route is None:
        raise NotImplementedError("vjp needs a function decorated with enzyme_jax_ir(pipeline_options=B200Pipeline(...))")
    if len(primals) == 4:
        x, weights, key_cache, value_cache = primals
        route.check_token_call(x, weights, key_cache, value_cache)
        plan = route._ensure(weights, True)
        out = route.decode_hidden(x, weights, key_cache, value_cache)

        def pullback_token(d_hidden: torch.Tensor):
            _, dx, packed, dkc, dvc = plan.token_vjp(x, key_cache, value_cache, d_hidden)
            leaves = plan.unpack_grads(packed)
            return dx, {k: leaves[k] for k in weights}, dkc, dvc

        return out, pullback_token
    if len(primals) != 2:
        raise NotImplementedError("vjp takes (fn, x, weights, key_cache, value_cache) or (fn, tokens, weights)")
    tokens, weights = primals
    route.check_sequence_call(tokens, weights)
    plan = route._ensure(weights, True)
    tok = tokens.to(plan.device, torch.int32).contiguous()
    saved = plan.new_saved(*tok.shape)
    logits = plan.forward(tok, saved=saved)

    def pullback(dlogits: torch.Tensor):
        grads = plan.backward(tok, dlogits.to(plan.device, torch.float32).contiguous(), saved, plan.new_grads())
        leaves = plan.unpack_grads(grads)
        return None, {k: leaves[k] for k in weights}

    return logits, pullback


FFI_TARGETS = ("enzymejax_b200_llama_pack", "enzymejax_b200_llama_fwd", "enzymejax_b200_llama_fwd_saved",
               "enzymejax_b200_llama_bwd", "enzymejax_b200_llama_unpack_grads", "enzymejax_b200_llama_decode_step",
               "enzymejax_b200_llama_token_fwd", "enzymejax_b200_llama_token_vjp")


def register_ffi_targets(jax_ffi=None) -> Tuple[str, ...]:
    """Registers the library's XLA typed-FFI handlers with JAX, once per process, the way the reference registers its
    own at import (primitives.py:32-40): every handler address from ``b200_ffi_handler`` is wrapped in a PyCapsule
    named ``xla._CUSTOM_CALL_TARGET`` and passed to ``jax.ffi.register_ffi_target(name, capsule, platform="CUDA")``.
    ``jax_ffi`` defaults to ``jax.ffi``.  Raises ``NotImplementedError`` where JAX is missing or the library was built
    without the XLA FFI headers."""
    import ctypes
    lib = _B.lib()
    if jax_ffi is None:
        try:
            import jax.ffi as jax_ffi  # type: ignore
        except Exception as exc:  # no JAX in this environment
            raise NotImplementedError(f"jax.ffi is not importable here ({exc}); the handlers cannot be registered") from exc
    if not lib.b200_ffi_available():
        raise NotImplementedError("the library was built without the XLA FFI headers (xla/ffi/api/ffi.h); rebuild it "
                                  "where jaxlib is installed")
    global _FFI_REGISTERED
    if _FFI_REGISTERED:
        return FFI_TARGETS
    capsule_new = ctypes.pythonapi.PyCapsule_New
    capsule_new.restype = ctypes.py_object
    capsule_new.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p]
    for name in FFI_TARGETS:
        addr = lib.b200_ffi_handler(name.encode())
        if not addr:
            raise NotImplementedError(f"the library has no handler named {name}")
        jax_ffi.register_ffi_target(name, capsule_new(addr, b"xla._CUSTOM_CALL_TARGET", None), platform="CUDA")
    _FFI_REGISTERED = True
    return FFI_TARGETS


_FFI_REGISTERED = False

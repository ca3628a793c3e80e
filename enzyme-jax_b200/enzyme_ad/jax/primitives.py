"""The reference's Python surface for the llama path, backed by the B200 library.

Mirrors the names of the reference's ``enzyme_ad.jax`` package
(``src/enzyme_ad/jax/__init__.py:1-12``): ``enzyme_jax_ir`` keeps its signature
(``primitives.py:1528``), the pipeline classes keep their methods
(``primitives.py:56-115``).  JAX is not installed where this runs, so the
decorated function takes and returns torch CUDA tensors; under JAX the same
routing sits behind ``jax.ffi.ffi_call`` and ``jax.custom_vjp``.

Only the llama path is implemented.  A function decorated with
``enzyme_jax_ir(pipeline_options=B200Pipeline(config))`` is recognised by its
arguments:

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
    def decode_hidden(self, x, weights, key_cache, value_cache):
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
    def forward_logits(self, tokens, weights, saved=None):
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
            if len(args) == 4 and isinstance(args[1], dict):
                return route.decode_hidden(*args)
            if len(args) == 2 and isinstance(args[1], dict) and not args[0].dtype.is_floating_point:
                return route.forward_logits(*args)
            raise NotImplementedError(
                "unrecognised call: expected (x, weights, key_cache, value_cache) or (tokens, weights)")

        wrapped._b200_route = route
        return wrapped

    return decorator


def vjp(fn: Callable, tokens: torch.Tensor, weights: Dict[str, torch.Tensor]) -> Tuple[torch.Tensor, Callable]:
    """``jax.vjp``-shaped helper for a decorated ``fn(tokens, weights)``: returns the
    logits and a function mapping a logits cotangent to the dict of weight
    gradients (what the reference's ``enzyme_vjp`` rule yields for the weight
    arguments, primitives.py:1381-1469)."""
    route: _LlamaRoute = getattr(fn, "_b200_route", None)
    if route is None:
        raise NotImplementedError("vjp needs a function decorated with enzyme_jax_ir(pipeline_options=B200Pipeline(...))")
    plan = route._ensure(weights, True)
    tok = tokens.to(plan.device, torch.int32).contiguous()
    saved = plan.new_saved(*tok.shape)
    logits = plan.forward(tok, saved=saved)

    def pullback(dlogits: torch.Tensor) -> Dict[str, torch.Tensor]:
        grads = plan.backward(tok, dlogits.to(plan.device, torch.float32).contiguous(), saved, plan.new_grads())
        leaves = plan.unpack_grads(grads)
        return {k: leaves[k] for k in weights}

    return logits, pullback

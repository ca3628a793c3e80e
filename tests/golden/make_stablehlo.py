"""Writes tests/golden/llama_forward_tiny.stablehlo.mlir: StableHLO text of the reference's llama ``forward``.

    python tests/golden/make_stablehlo.py <path of the reference tree>

JAX is not installable where this runs, so the text cannot come from ``jax.jit(fn).lower(...).as_text()`` (the text
the reference hands to its pass pipeline, src/enzyme_ad/jax/primitives.py:593-601).  Instead the reference's own
``forward`` source (test/llama.py:35-238) is executed, unmodified, with a recording stand-in registered as
``jax.numpy``: every array operation the source performs on an argument is written down as the StableHLO operation
JAX lowers it to (``x.dot(x)`` and ``@`` -> ``stablehlo.dot_general``, ``jnp.einsum`` -> ``dot_general`` with batching /
contracting dimensions, indexing -> ``slice`` + ``reshape``, ``jnp.max`` -> ``reduce`` with ``maximum``, Python ``sum`` ->
a chain of ``add``, ``jnp.append`` / ``concatenate`` -> ``concatenate``, scalars -> ``constant`` + ``broadcast_in_dim``).
Values the source computes from Python numbers only (the rotation table: ``pos`` is ``key_cache.shape[1]``, a Python
int) stay numpy arrays and appear as ``stablehlo.constant``, as they do under JAX.  Arguments are ordered as JAX flattens
``(x, weights, key_cache, value_cache)``: x, the weight leaves in sorted-key order, the two caches.

The fixture exists to test the text matcher (enzyme_ad/jax/hlo_matcher.py); its operation graph is the reference's,
its spelling is this file's.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

TINY = dict(dim=8, hidden_dim=16, n_layers=2, n_heads=2, n_kv_heads=2, vocab_size=32, seq_len=16)
POS = 2  # rows already in the caches


class Emitter:
    def __init__(self):
        self.lines = []
        self.n = 0
        self.ncst = 0

    def fresh(self):
        name = f"%{self.n}"
        self.n += 1
        return name

    def ttype(self, shape):
        return "tensor<" + "".join(f"{int(d)}x" for d in shape) + "f32>"

    def constant(self, value):
        arr = np.asarray(value, dtype=np.float32)
        name = "%cst" if self.ncst == 0 else f"%cst_{self.ncst - 1}"
        self.ncst += 1

        def lit(a):
            if a.ndim == 0:
                return f"{float(a):.6e}"
            return "[" + ", ".join(lit(x) for x in a) + "]"

        self.lines.append(f"    {name} = stablehlo.constant dense<{lit(arr)}> : {self.ttype(arr.shape)}")
        return Tr(self, name, arr.shape)

    def op(self, text, shape):
        name = self.fresh()
        self.lines.append(f"    {name} = {text}")
        return Tr(self, name, tuple(int(d) for d in shape))


class Tr:
    """A traced f32 array: SSA name + static shape."""
    __array_priority__ = 1000

    def __init__(self, em: Emitter, name: str, shape):
        self.em, self.name, self.shape = em, name, tuple(int(d) for d in shape)

    @property
    def ndim(self):
        return len(self.shape)

    def __len__(self):
        return self.shape[0]

    def __iter__(self):
        return (self[i] for i in range(self.shape[0]))

    # ---- helpers ---------------------------------------------------------------------------------
    def _lift(self, other):
        """other as a traced array of this array's shape (scalars are broadcast, arrays become constants)."""
        if isinstance(other, Tr):
            if other.shape == self.shape:
                return other
            if other.shape == ():
                return other.broadcast_to(self.shape)
            raise NotImplementedError(f"broadcast {other.shape} -> {self.shape}")
        arr = np.asarray(other, dtype=np.float32)
        c = self.em.constant(arr)
        return c if arr.shape == self.shape else c.broadcast_to(self.shape)

    def broadcast_to(self, shape):
        assert self.shape == ()
        if tuple(shape) == ():
            return self
        t = self.em.ttype(shape)
        return self.em.op(f"stablehlo.broadcast_in_dim {self.name}, dims = [] : ({self.em.ttype(())}) -> {t}", shape)

    def _bin(self, opname, other, swap=False):
        rhs = self._lift(other)
        a, b = (rhs, self) if swap else (self, rhs)
        return self.em.op(f"stablehlo.{opname} {a.name}, {b.name} : {self.em.ttype(self.shape)}", self.shape)

    def _un(self, opname):
        return self.em.op(f"stablehlo.{opname} {self.name} : {self.em.ttype(self.shape)}", self.shape)

    # ---- arithmetic ------------------------------------------------------------------------------
    def __add__(self, o): return self._bin("add", o)
    def __radd__(self, o): return self._bin("add", o, swap=True)
    def __iadd__(self, o): return self._bin("add", o)
    def __sub__(self, o): return self._bin("subtract", o)
    def __rsub__(self, o): return self._bin("subtract", o, swap=True)
    def __mul__(self, o): return self._bin("multiply", o)
    def __rmul__(self, o): return self._bin("multiply", o, swap=True)
    def __truediv__(self, o): return self._bin("divide", o)
    def __rtruediv__(self, o): return self._bin("divide", o, swap=True)
    def __neg__(self): return self._un("negate")

    # ---- shape ops -------------------------------------------------------------------------------
    def reshape(self, shape):
        shape = tuple(int(d) for d in shape)
        if shape == self.shape:
            return self
        return self.em.op(f"stablehlo.reshape {self.name} : ({self.em.ttype(self.shape)}) -> {self.em.ttype(shape)}", shape)

    def __getitem__(self, idx):
        if not isinstance(idx, tuple):
            idx = (idx,)
        idx = idx + (slice(None),) * (self.ndim - len(idx))
        lo, hi, keep = [], [], []
        for d, (i, n) in enumerate(zip(idx, self.shape)):
            if isinstance(i, slice):
                a, b, st = i.indices(n)
                assert st == 1
                lo.append(a); hi.append(max(a, b)); keep.append(True)
            else:
                i = int(i) + (n if int(i) < 0 else 0)
                lo.append(i); hi.append(i + 1); keep.append(False)
        out_shape = tuple(h - l for l, h in zip(lo, hi))
        res = self
        if out_shape != self.shape:
            rng = ", ".join(f"{l}:{h}" for l, h in zip(lo, hi))
            res = self.em.op(f"stablehlo.slice {self.name} [{rng}] : ({self.em.ttype(self.shape)}) -> {self.em.ttype(out_shape)}",
                             out_shape)
        return res.reshape(tuple(s for s, k in zip(out_shape, keep) if k))

    # ---- contractions ----------------------------------------------------------------------------
    def dot(self, other):
        return dot_general(self, other, [], [], [self.ndim - 1], [0])

    def __matmul__(self, other):
        return dot_general(self, other, [], [], [self.ndim - 1], [0])


def _as_tr(em, v):
    return v if isinstance(v, Tr) else em.constant(v)


def dot_general(a, b, batch_a, batch_b, con_a, con_b):
    em = a.em if isinstance(a, Tr) else b.em
    a, b = _as_tr(em, a), _as_tr(em, b)
    free_a = [d for d in range(a.ndim) if d not in batch_a and d not in con_a]
    free_b = [d for d in range(b.ndim) if d not in batch_b and d not in con_b]
    shape = [a.shape[d] for d in batch_a] + [a.shape[d] for d in free_a] + [b.shape[d] for d in free_b]
    attrs = []
    if batch_a:
        attrs.append(f"batching_dims = {list(batch_a)} x {list(batch_b)}")
    attrs.append(f"contracting_dims = {list(con_a)} x {list(con_b)}")
    attrs.append("precision = [DEFAULT, DEFAULT]")
    return em.op(f"stablehlo.dot_general {a.name}, {b.name}, {', '.join(attrs)} : "
                 f"({em.ttype(a.shape)}, {em.ttype(b.shape)}) -> {em.ttype(shape)}", shape)


def make_jnp(em: Emitter):
    """The subset of jax.numpy the reference's forward uses, recording operations on traced arrays."""
    m = types.ModuleType("jax.numpy")

    def unary(np_fn, hlo):
        def f(x):
            return x._un(hlo) if isinstance(x, Tr) else np_fn(x)
        return f

    m.sqrt = unary(np.sqrt, "sqrt")
    m.exp = unary(np.exp, "exponential")
    m.cos = unary(np.cos, "cosine")
    m.sin = unary(np.sin, "sine")
    m.power = np.power      # only ever called on Python numbers (test/llama.py:130)
    m.eye = np.eye
    m.array = np.array      # only ever called on values computed from Python numbers (the rotation table)
    m.zeros = np.zeros

    def jmax(x):
        if not isinstance(x, Tr):
            return np.max(x)
        init = em.constant(-np.inf)
        dims = list(range(x.ndim))
        return em.op(f"stablehlo.reduce({x.name} init: {init.name}) applies stablehlo.maximum across dimensions = {dims} : "
                     f"({em.ttype(x.shape)}, {em.ttype(())}) -> {em.ttype(())}", ())

    m.max = jmax

    def reshape(x, shape):
        return x.reshape(shape) if isinstance(x, Tr) else np.reshape(x, shape)

    m.reshape = reshape

    def concatenate(parts, axis=0):
        parts = [_as_tr(em, p) for p in parts]
        if axis is None:
            parts = [p.reshape((int(np.prod(p.shape)),)) for p in parts]
            axis = 0
        shape = list(parts[0].shape)
        shape[axis] = sum(p.shape[axis] for p in parts)
        return em.op(f"stablehlo.concatenate {', '.join(p.name for p in parts)}, dim = {axis} : "
                     f"({', '.join(em.ttype(p.shape) for p in parts)}) -> {em.ttype(shape)}", shape)

    m.concatenate = concatenate
    m.append = lambda a, b, axis=None: concatenate([a, b], axis=axis)

    def einsum(spec, a, b):
        lhs, out = spec.replace(" ", "").split("->")
        la, lb = lhs.split(",")
        batch = [c for c in la if c in lb and c in out]
        con = [c for c in la if c in lb and c not in out]
        res = dot_general(a, b, [la.index(c) for c in batch], [lb.index(c) for c in batch],
                          [la.index(c) for c in con], [lb.index(c) for c in con])
        order = batch + [c for c in la if c not in batch and c not in con] + [c for c in lb if c not in batch and c not in con]
        assert "".join(order) == out, "a transpose would be needed; the reference's einsums need none"
        return res

    m.einsum = einsum
    return m


def load_reference_forward(ref_root: str, jnp_module):
    """The reference's test/llama.py with `jax.numpy` bound to `jnp_module` (its other imports are never reached by
    `forward`)."""
    jax_mod = types.ModuleType("jax")
    jax_mod.numpy = jnp_module
    stubs = {"jax": jax_mod, "jax.numpy": jnp_module, "jax.random": types.ModuleType("jax.random"),
             "jax.lax": types.ModuleType("jax.lax")}
    absl = types.ModuleType("absl")
    absltest = types.ModuleType("absl.testing.absltest")
    absltest.TestCase = object
    absltest.main = lambda *a, **k: None
    absl_testing = types.ModuleType("absl.testing")
    absl_testing.absltest = absltest
    absl.testing = absl_testing
    stubs.update({"absl": absl, "absl.testing": absl_testing, "absl.testing.absltest": absltest})
    tu = types.ModuleType("test_utils")
    tu.EnzymeJaxTest = object
    tu.pipelines = lambda: []
    tu.CurBackends = []
    stubs["test_utils"] = tu
    saved = {k: sys.modules.get(k) for k in stubs}
    sys.modules.update(stubs)
    try:
        spec = importlib.util.spec_from_file_location("reference_llama_for_stablehlo", os.path.join(ref_root, "test", "llama.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod, saved
    except Exception:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
        raise


def weight_shapes(cfg):
    L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    return {"rms_att_weight": (L, d), "rms_ffn_weight": (L, d), "rms_final_weight": (d,), "w1": (L, h, d),
            "w2": (L, d, h), "w3": (L, h, d), "wcls": (V, d), "wk": (L, d, d), "wo": (L, d, d), "wq": (L, d, d),
            "wv": (L, d, d)}


def emit(ref_root: str, cfg=TINY, pos=POS, drop_unused=False) -> str:
    em = Emitter()
    jnp = make_jnp(em)
    mod, saved = load_reference_forward(ref_root, jnp)
    try:
        shapes = weight_shapes(cfg)
        arg_shapes = [("x", (cfg["dim"],))] + [(k, shapes[k]) for k in sorted(shapes)] + \
                     [("key_cache", (cfg["n_layers"], pos, cfg["dim"])), ("value_cache", (cfg["n_layers"], pos, cfg["dim"]))]
        if drop_unused:  # what JAX's dead-argument elimination leaves (the reference emulates it, primitives.py:1550-1569)
            arg_shapes = [a for a in arg_shapes if a[0] != "wcls"]
        args = {}
        for i, (name, shape) in enumerate(arg_shapes):
            args[name] = Tr(em, f"%arg{i}", shape)
        weights = {k: args.get(k, Tr(em, "%dropped", shapes[k])) for k in shapes}
        out = mod.forward(args["x"], cfg, weights, args["key_cache"], args["value_cache"])
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
    sig = ", ".join(f"%arg{i}: {em.ttype(s)}" for i, (_, s) in enumerate(arg_shapes))
    head = ["module @jit_sfn attributes {mhlo.num_partitions = 1 : i32, mhlo.num_replicas = 1 : i32} {",
            f"  func.func public @main({sig}) -> ({em.ttype(out.shape)} {{jax.result_info = \"\"}}) {{"]
    tail = [f"    return {out.name} : {em.ttype(out.shape)}", "  }", "}"]
    return "\n".join(head + em.lines + tail) + "\n"


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_stablehlo.py <path of the reference tree>")
    for name, drop in (("llama_forward_tiny.stablehlo.mlir", False), ("llama_forward_tiny_dce.stablehlo.mlir", True)):
        text = emit(sys.argv[1], drop_unused=drop)
        path = os.path.join(HERE, name)
        with open(path, "w") as f:
            f.write(text)
        print("wrote", path, len(text.splitlines()), "lines")


if __name__ == "__main__":
    main()

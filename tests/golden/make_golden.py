"""Generate golden vectors from the reference's own ``forward`` source.

The reference (``test/llama.py`` in the EnzymeAD/Enzyme-JAX tree) is written
against ``jax.numpy``; JAX is not installable in the build container, so this
script loads the reference file unmodified with ``numpy`` registered under the
name ``jax.numpy`` (every ``jnp`` call the file makes -- sqrt, max, exp,
power, cos, sin, array, eye, reshape, einsum, append, concatenate -- has the
same name and meaning in numpy) and stubs for the two harness imports at the
top of the file.  The reference's ``forward`` is then executed as is.

Run from the repository root, with the reference tree mounted:

    python tests/golden/make_golden.py /path/to/reference

It writes ``tests/golden/llama_golden.npz``.  The inputs are regenerated from
seeds by the tests; only reference OUTPUTS (and the seeds) are stored.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def load_reference_llama(ref_root: str):
    jax = types.ModuleType("jax")
    jax.numpy = np
    sys.modules.setdefault("jax", jax)
    sys.modules.setdefault("jax.numpy", np)
    absl = types.ModuleType("absl")
    absl_testing = types.ModuleType("absl.testing")
    absltest = types.ModuleType("absl.testing.absltest")
    absltest.TestCase = object
    absl_testing.absltest = absltest
    absl.testing = absl_testing
    sys.modules.setdefault("absl", absl)
    sys.modules.setdefault("absl.testing", absl_testing)
    sys.modules.setdefault("absl.testing.absltest", absltest)
    tu = types.ModuleType("test_utils")
    tu.EnzymeJaxTest = object
    tu.CurBackends = []
    tu.pipelines = lambda: []
    sys.modules.setdefault("test_utils", tu)
    spec = importlib.util.spec_from_file_location("ref_llama", os.path.join(ref_root, "test", "llama.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def uniform_weights(cfg, seed, dtype):
    """uniform[0,1) leaves like the reference's setUp (test/llama.py:283-286),
    drawn from numpy's PCG64 (JAX's threefry stream is not reproducible here)."""
    from oracle import llama_ref as O
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in sorted(O.weight_shapes(cfg).items()):
        w[name] = rng.random(shape).astype(dtype)
    return w, rng


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <path of the reference tree>")
    ref_root = sys.argv[1]
    ref = load_reference_llama(ref_root)
    import torch
    from oracle import llama_ref as O

    out = {}

    # Case A: the shipped test's shape and cache (dim 288, pos=1 zero cache), fp32 and fp64.
    cfg = O.CONFIGS["c1"]
    kv_dim = cfg["dim"]
    for tag, dt in (("f32", np.float32), ("f64", np.float64)):
        w, rng = uniform_weights(cfg, 11, dt)
        x = rng.random(cfg["dim"]).astype(dt)
        kc = np.zeros((cfg["n_layers"], 1, kv_dim), dt)
        out[f"A_{tag}"] = ref.forward(x.copy(), cfg, w, kc, kc.copy())

    # Case B: small shape, random cache of 5 rows, N(0,0.02)-like weights, fp64.
    cfg = O.CONFIGS["tiny"]
    w = O.to_numpy(O.make_weights(cfg, 5, torch.float64, std=0.2, gains_one=False))
    rng = np.random.default_rng(21)
    x = rng.standard_normal(cfg["dim"])
    kc = rng.standard_normal((cfg["n_layers"], 5, cfg["dim"]))
    vc = rng.standard_normal((cfg["n_layers"], 5, cfg["dim"]))
    out["B_f64"] = ref.forward(x.copy(), cfg, w, kc, vc)

    # Case C: empty cache (pos=0).
    kc0 = np.zeros((cfg["n_layers"], 0, cfg["dim"]))
    out["C_f64"] = ref.forward(x.copy(), cfg, w, kc0, kc0.copy())

    # Case D: full sequence.  Level 1 provides the embedding rows and the K/V
    # rows of the earlier positions; the reference forward is run per token on
    # those caches and its hidden state is stored.
    tokens = O.make_tokens(cfg, 2, 12, 3)
    wt = O.make_weights(cfg, 5, torch.float64, std=0.2, gains_one=False)
    _, aux = O.forward_sequence(tokens, cfg, wt, return_aux=True)
    K = aux["k"].numpy()   # [L,B,S,d]
    V = aux["v"].numpy()
    E = w["token_embedding_table"]
    hid = np.zeros((2, 12, cfg["dim"]))
    for b in range(2):
        for t in range(12):
            hid[b, t] = ref.forward(E[int(tokens[b, t])].copy(), cfg, w, K[:, b, :t].copy(), V[:, b, :t].copy())
    out["D_hidden_f64"] = hid

    path = os.path.join(HERE, "llama_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()

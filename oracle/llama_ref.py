"""CPU oracle for the llama forward / VJP hot path.  TEST INFRASTRUCTURE ONLY.

This module is a checker: only the test-suite, the smoke entry and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.
The product (the CUDA library and its Python host layer) never does.

It restates, in numpy / torch-CPU, the model of the reference's
``test/llama.py``:

* ``rmsnorm``            follows test/llama.py:6-10   (eps inside the sqrt)
* ``softmax``            follows test/llama.py:13-18  (max-shifted)
* ``silu``               follows test/llama.py:21-28  (x / (1 + exp(-x)))
* ``forward_token``      follows test/llama.py:35-238 (Level 0: one token, a
  cache of ``pos`` rows per layer, returns the final-normed hidden state)
* ``forward_sequence``   Level 1: full causal sequence with embedding lookup
  and the logits projection (both commented out in the reference at
  test/llama.py:109-113 and :236; the benchmark configs add them back)
* ``vjp_sequence``       Level 2: reverse mode of Level 1 by torch autograd in
  the requested precision; the per-op rules it must agree with are the
  reference's Implementations/HLODerivatives.td:964-1339 (dot_general, mul,
  div, exp, rsqrt ...) and StableHLOAutoDiffOpInterfaceImpl.cpp:1474-2070.

Parity pin: the arithmetic of the reference runs inside XLA, which is not
vendored in the reference tree and is not installable here.  Level 0 and
Level 1 are pinned against the reference's own ``forward`` source executed
with numpy standing in for ``jax.numpy`` (tests/golden/make_golden.py); the
XLA execution itself is unpinned ("parity unpinned" for XLA's rounding).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

WEIGHT_KEYS = (
    "rms_att_weight", "rms_ffn_weight", "rms_final_weight", "token_embedding_table",
    "w1", "w2", "w3", "wcls", "wk", "wo", "wq", "wv",
)

CONFIGS = {
    # llama2.c "stories15M" shape used by the reference test (test/llama.py:246-254)
    "c1": dict(dim=288, hidden_dim=768, n_layers=6, n_heads=6, n_kv_heads=6, vocab_size=32000, seq_len=256),
    "c2": dict(dim=768, hidden_dim=2048, n_layers=12, n_heads=12, n_kv_heads=12, vocab_size=32000, seq_len=1024),
    "c4": dict(dim=4096, hidden_dim=11008, n_layers=32, n_heads=32, n_kv_heads=32, vocab_size=32000, seq_len=2048),
    "tiny": dict(dim=64, hidden_dim=128, n_layers=2, n_heads=2, n_kv_heads=2, vocab_size=96, seq_len=16),
}

ROPE_THETA = 10000.0
RMS_EPS = 1e-5


def weight_shapes(cfg) -> Dict[str, Tuple[int, ...]]:
    """Leaf names and shapes (test/llama.py:270-282, plus the embedding leaf
    named in the commented-out lines test/llama.py:109-112)."""
    L, d, h, V = cfg["n_layers"], cfg["dim"], cfg["hidden_dim"], cfg["vocab_size"]
    kv = d // cfg["n_heads"] * cfg["n_kv_heads"]
    return {
        "rms_att_weight": (L, d), "rms_ffn_weight": (L, d), "rms_final_weight": (d,),
        "token_embedding_table": (V, d),
        "w1": (L, h, d), "w2": (L, d, h), "w3": (L, h, d), "wcls": (V, d),
        "wk": (L, kv, d), "wo": (L, d, d), "wq": (L, d, d), "wv": (L, kv, d),
    }


def make_weights(cfg, seed: int, dtype=torch.float32, std: float = 0.02, gains_one: bool = True):
    """Seeded synthetic weights: matrices ~N(0, std^2), RMSNorm gains = 1 (or
    1 + N(0, 0.1^2) when ``gains_one`` is False, to exercise the gain path)."""
    out = {}
    for i, (name, shape) in enumerate(sorted(weight_shapes(cfg).items())):
        g = torch.Generator().manual_seed(seed * 1000 + i)
        if name.startswith("rms_"):
            t = torch.ones(shape, dtype=torch.float32)
            if not gains_one:
                t = t + 0.1 * torch.randn(shape, generator=g, dtype=torch.float32)
        else:
            t = torch.randn(shape, generator=g, dtype=torch.float32) * std
        out[name] = t.to(dtype)
    return out


def make_tokens(cfg, batch: int, seq: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed * 1000 + 977)
    return torch.randint(0, cfg["vocab_size"], (batch, seq), generator=g, dtype=torch.int64)


# --------------------------------------------------------------------------
# Level 0: one token against a cache (numpy), the reference's signature.
# --------------------------------------------------------------------------

def rmsnorm(x, weight):
    ss = 1.0 / np.sqrt(np.dot(x, x) / x.shape[0] + RMS_EPS)
    return weight * x * ss


def softmax(x):
    e = np.exp(x - np.max(x))
    return e / e.sum()


def silu(x):
    return x * (1.0 / (1.0 + np.exp(-x)))


def rope_angles(pos, head_size: int, n_pairs: int, dtype=np.float64):
    """cos/sin for pair index j in [0, n_pairs): the pair covers elements
    (2j, 2j+1) and its frequency is 10000^(-((2j) mod hs)/hs)
    (test/llama.py:129-135)."""
    i = (2 * np.arange(n_pairs)) % head_size
    freq = 1.0 / np.power(np.asarray(ROPE_THETA, dtype=dtype), i.astype(dtype) / head_size)
    ang = np.asarray(pos, dtype=dtype)[..., None] * freq
    return np.cos(ang), np.sin(ang)


def rotate_pairs(vec, c, s):
    """Rotate adjacent pairs (2j, 2j+1) of the last axis by the 2x2 matrix
    [[c, -s], [s, c]] (test/llama.py:137, 161-168)."""
    even, odd = vec[..., 0::2], vec[..., 1::2]
    out = np.empty_like(vec)
    out[..., 0::2] = c * even - s * odd
    out[..., 1::2] = s * even + c * odd
    return out


def forward_token(x, config, weights, key_cache, value_cache, return_kv: bool = False):
    """One decode step.  ``key_cache``/``value_cache`` are [L, pos, kv_dim];
    the new token sits at position ``pos`` (test/llama.py:38).  Returns the
    final-normed hidden state [dim] like the reference (test/llama.py:235-238).
    As in the reference, n_kv_heads must equal n_heads (the reshape at
    test/llama.py:162 requires kv_dim == dim)."""
    x = np.array(x, copy=True)
    dt = x.dtype
    pos = key_cache.shape[1]
    L, d, H = config["n_layers"], config["dim"], config["n_heads"]
    hs = d // H
    kv_mul = H // config["n_kv_heads"]
    c, s = rope_angles(np.asarray(pos), hs, d // 2, dtype=dt)
    new_k, new_v = [], []
    for l in range(L):
        xb = rmsnorm(x, weights["rms_att_weight"][l])
        q = weights["wq"][l] @ xb
        k = weights["wk"][l] @ xb
        v = weights["wv"][l] @ xb
        q = rotate_pairs(q, c, s)
        k = rotate_pairs(k, c, s)
        kc = np.concatenate([key_cache[l], k[None, :]], axis=0)      # new row last (:170-175)
        vc = np.concatenate([value_cache[l], v[None, :]], axis=0)
        new_k.append(k)
        new_v.append(v)
        heads = []
        for h in range(H):
            kvh = h // kv_mul
            sl = slice(kvh * hs, (kvh + 1) * hs)
            att = kc[:, sl] @ q[h * hs:(h + 1) * hs]
            att = softmax(att / np.sqrt(np.asarray(hs, dtype=dt)))
            heads.append(att @ vc[:, sl])
        x = x + weights["wo"][l] @ np.concatenate(heads)
        xb = rmsnorm(x, weights["rms_ffn_weight"][l])
        hb = silu(weights["w1"][l] @ xb) * (weights["w3"][l] @ xb)
        x = x + weights["w2"][l] @ hb
    out = rmsnorm(x, weights["rms_final_weight"])
    if return_kv:
        return out, np.stack(new_k), np.stack(new_v)
    return out


# --------------------------------------------------------------------------
# Level 1 / Level 2: full sequence (torch CPU, differentiable).
# --------------------------------------------------------------------------

def _t_rmsnorm(x, g):
    r = torch.rsqrt((x * x).mean(dim=-1, keepdim=True) + RMS_EPS)
    return g * x * r


def _t_rope_table(positions: torch.Tensor, hs: int, dtype):
    j2 = torch.arange(0, hs, 2, dtype=torch.float64)
    freq = 1.0 / torch.pow(torch.tensor(ROPE_THETA, dtype=torch.float64), j2 / hs)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def _t_rotate(v, c, s):
    # v [B,S,H,hs]; c,s [S,hs/2]
    ev, od = v[..., 0::2], v[..., 1::2]
    c = c[None, :, None, :]
    s = s[None, :, None, :]
    return torch.stack((c * ev - s * od, s * ev + c * od), dim=-1).flatten(-2)


def forward_sequence(tokens: torch.Tensor, cfg, w, *, past_k: Optional[torch.Tensor] = None,
                     past_v: Optional[torch.Tensor] = None, return_aux: bool = False):
    """Causal forward over tokens [B,S] -> logits [B,S,V].

    ``past_k``/``past_v`` [L,B,P,d] (already rotated keys) extend the context
    to the left: token s then sits at position P+s.  Precision is that of the
    weight tensors."""
    B, S = tokens.shape
    L, d, H = cfg["n_layers"], cfg["dim"], cfg["n_heads"]
    hs = d // H
    dt = w["wq"].dtype
    P = 0 if past_k is None else past_k.shape[2]
    c, s = _t_rope_table(torch.arange(P, P + S), hs, dt)
    x = w["token_embedding_table"][tokens]
    mask = torch.ones(S, P + S, dtype=torch.bool).tril(diagonal=P)
    aux = {"k": [], "v": []}
    for l in range(L):
        xb = _t_rmsnorm(x, w["rms_att_weight"][l])
        q = (xb @ w["wq"][l].T).view(B, S, H, hs)
        k = (xb @ w["wk"][l].T).view(B, S, H, hs)
        v = (xb @ w["wv"][l].T).view(B, S, H, hs)
        q = _t_rotate(q, c, s)
        k = _t_rotate(k, c, s)
        aux["k"].append(k.reshape(B, S, d))
        aux["v"].append(v.reshape(B, S, d))
        if P:
            k = torch.cat([past_k[l].view(B, P, H, hs), k], dim=1)
            v = torch.cat([past_v[l].view(B, P, H, hs), v], dim=1)
        att = torch.einsum("bthe,buhe->bhtu", q, k) / math.sqrt(hs)
        att = att.masked_fill(~mask, float("-inf"))
        att = torch.softmax(att, dim=-1)
        o = torch.einsum("bhtu,buhe->bthe", att, v).reshape(B, S, d)
        x = x + o @ w["wo"][l].T
        xb = _t_rmsnorm(x, w["rms_ffn_weight"][l])
        a = xb @ w["w1"][l].T
        hb = a * torch.sigmoid(a) * (xb @ w["w3"][l].T)
        x = x + hb @ w["w2"][l].T
    xf = _t_rmsnorm(x, w["rms_final_weight"])
    logits = xf @ w["wcls"].T
    if return_aux:
        aux["xf"] = xf
        aux["k"] = torch.stack(aux["k"])
        aux["v"] = torch.stack(aux["v"])
        return logits, aux
    return logits


def vjp_sequence(tokens, cfg, w, dlogits):
    """Gradients of <logits, dlogits> with respect to every weight leaf."""
    leaves = {k: v.detach().clone().requires_grad_(True) for k, v in w.items()}
    logits = forward_sequence(tokens, cfg, leaves)
    logits.backward(dlogits.to(logits.dtype))
    return logits.detach(), {k: (v.grad if v.grad is not None else torch.zeros_like(v)) for k, v in leaves.items()}


def jvp_sequence(tokens, cfg, w, dw):
    """Forward mode of Level 1: (logits, tangent of the logits) for tangents ``dw`` of the weight leaves (missing
    leaves count as zero), by torch's forward-mode AD; the reference's harness computes the same with jax.jvp
    (test/test_utils.py:689-735)."""
    import torch.autograd.forward_ad as fwAD
    with fwAD.dual_level():
        dual = {k: fwAD.make_dual(v, dw[k].to(v.dtype) if k in dw else torch.zeros_like(v)) for k, v in w.items()}
        out = forward_sequence(tokens, cfg, dual)
        primal, tangent = fwAD.unpack_dual(out)
        return primal.detach(), (tangent if tangent is not None else torch.zeros_like(primal)).detach()


def jvp_token(x, cfg, w, key_cache, value_cache, dx, dw, d_key_cache, d_value_cache):
    """Forward mode of the reference's own call with tangents for all inputs (jax.jvp(fn, ins, dins),
    test/test_utils.py:689-735): returns (hidden, tangent of hidden)."""
    import torch.autograd.forward_ad as fwAD
    dt = w["wq"].dtype
    tokens = torch.zeros(1, 1, dtype=torch.int64)
    with fwAD.dual_level():
        dual = {k: fwAD.make_dual(v, dw[k].to(dt) if k in dw else torch.zeros_like(v)) for k, v in w.items()
                if k != "token_embedding_table"}
        dual["token_embedding_table"] = fwAD.make_dual(x.to(dt), dx.to(dt))[None, :]
        pk = fwAD.make_dual(key_cache.to(dt), d_key_cache.to(dt))[:, None] if key_cache.shape[1] else None
        pv = fwAD.make_dual(value_cache.to(dt), d_value_cache.to(dt))[:, None] if value_cache.shape[1] else None
        _, aux = forward_sequence(tokens, cfg, dual, past_k=pk, past_v=pv, return_aux=True)
        primal, tangent = fwAD.unpack_dual(aux["xf"][0, 0])
        return primal.detach(), tangent.detach()


def vjp_token(x, cfg, w, key_cache, value_cache, d_hidden):
    """Reverse mode of the reference's own call, forward(x, weights, key_cache, value_cache) -> hidden
    (test/llama.py:35-238), with respect to ALL inputs, as the reference's test differentiates it
    (test/llama.py:315-317, test/test_utils.py:505-514).  x [d]; caches [L, pos, d]; returns
    (hidden, dx, {leaf: grad}, d_key_cache, d_value_cache).  Level 1 serves: a one-row embedding table holding x
    turns the residual vector into a differentiable input; wcls and the real embedding table receive zero."""
    dt = w["wq"].dtype
    leaves = {k: v.detach().clone().requires_grad_(True) for k, v in w.items() if k != "token_embedding_table"}
    xin = x.detach().clone().to(dt).requires_grad_(True)
    kc = key_cache.detach().clone().to(dt).requires_grad_(True)
    vc = value_cache.detach().clone().to(dt).requires_grad_(True)
    full = dict(leaves, token_embedding_table=xin[None, :])
    tokens = torch.zeros(1, 1, dtype=torch.int64)
    _, aux = forward_sequence(tokens, cfg, full, past_k=kc[:, None] if kc.shape[1] else None,
                              past_v=vc[:, None] if vc.shape[1] else None, return_aux=True)
    hidden = aux["xf"][0, 0]
    hidden.backward(d_hidden.to(dt))
    grads = {k: (v.grad if v.grad is not None else torch.zeros_like(v)) for k, v in leaves.items()}
    zero = lambda t: torch.zeros_like(t) if t.grad is None else t.grad
    return hidden.detach(), zero(xin), grads, zero(kc), zero(vc)


def cast_weights(w, dtype):
    return {k: v.to(dtype) for k, v in w.items()}


def to_numpy(w):
    return {k: v.detach().cpu().numpy() for k, v in w.items()}

"""The CPU oracle against the golden vectors produced by the reference's own
``forward`` source (tests/golden/make_golden.py) and against itself."""
import os

import numpy as np
import pytest
import torch

from oracle import llama_ref as O

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "llama_golden.npz"))


def _uniform_weights(cfg, seed, dtype):
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in sorted(O.weight_shapes(cfg).items()):
        w[name] = rng.random(shape).astype(dtype)
    return w, rng


@pytest.mark.parametrize("tag,dt,tol", [("f32", np.float32, 2e-5), ("f64", np.float64, 1e-12)])
def test_level0_shipped_shape(tag, dt, tol):
    cfg = O.CONFIGS["c1"]
    w, rng = _uniform_weights(cfg, 11, dt)
    x = rng.random(cfg["dim"]).astype(dt)
    kc = np.zeros((cfg["n_layers"], 1, cfg["dim"]), dt)
    got = O.forward_token(x, cfg, w, kc, kc.copy())
    np.testing.assert_allclose(got, GOLD[f"A_{tag}"], rtol=tol, atol=tol)


def _tiny_case():
    cfg = O.CONFIGS["tiny"]
    wt = O.make_weights(cfg, 5, torch.float64, std=0.2, gains_one=False)
    w = O.to_numpy(wt)
    rng = np.random.default_rng(21)
    x = rng.standard_normal(cfg["dim"])
    kc = rng.standard_normal((cfg["n_layers"], 5, cfg["dim"]))
    vc = rng.standard_normal((cfg["n_layers"], 5, cfg["dim"]))
    return cfg, wt, w, x, kc, vc


def test_level0_random_cache_and_empty_cache():
    cfg, _, w, x, kc, vc = _tiny_case()
    np.testing.assert_allclose(O.forward_token(x, cfg, w, kc, vc), GOLD["B_f64"], rtol=1e-12, atol=1e-12)
    e = np.zeros((cfg["n_layers"], 0, cfg["dim"]))
    np.testing.assert_allclose(O.forward_token(x, cfg, w, e, e.copy()), GOLD["C_f64"], rtol=1e-12, atol=1e-12)


def test_level1_hidden_matches_reference_per_token():
    cfg, wt, _, _, _, _ = _tiny_case()
    tokens = O.make_tokens(cfg, 2, 12, 3)
    _, aux = O.forward_sequence(tokens, cfg, wt, return_aux=True)
    np.testing.assert_allclose(aux["xf"].numpy(), GOLD["D_hidden_f64"], rtol=1e-10, atol=1e-11)


def test_level1_equals_level0_iterated():
    cfg, wt, w, _, _, _ = _tiny_case()
    tokens = O.make_tokens(cfg, 1, 9, 8)
    logits, aux = O.forward_sequence(tokens, cfg, wt, return_aux=True)
    L, d = cfg["n_layers"], cfg["dim"]
    kc = np.zeros((L, 0, d))
    vc = np.zeros((L, 0, d))
    for t in range(9):
        x = w["token_embedding_table"][int(tokens[0, t])]
        h, nk, nv = O.forward_token(x, cfg, w, kc, vc, return_kv=True)
        np.testing.assert_allclose(h, aux["xf"][0, t].numpy(), rtol=1e-10, atol=1e-11)
        np.testing.assert_allclose(w["wcls"] @ h, logits[0, t].numpy(), rtol=1e-9, atol=1e-10)
        kc = np.concatenate([kc, nk[:, None, :]], axis=1)
        vc = np.concatenate([vc, nv[:, None, :]], axis=1)


def test_level1_past_cache_equals_full_sequence():
    cfg, wt, _, _, _, _ = _tiny_case()
    tokens = O.make_tokens(cfg, 2, 10, 4)
    full, aux = O.forward_sequence(tokens, cfg, wt, return_aux=True)
    P = 7
    part = O.forward_sequence(tokens[:, P:], cfg, wt, past_k=aux["k"][:, :, :P], past_v=aux["v"][:, :, :P])
    np.testing.assert_allclose(part.numpy(), full[:, P:].numpy(), rtol=1e-10, atol=1e-11)


def test_level2_vjp_matches_finite_differences():
    cfg, wt, _, _, _, _ = _tiny_case()
    tokens = O.make_tokens(cfg, 1, 6, 2)
    g = torch.Generator().manual_seed(0)
    dlogits = torch.randn(1, 6, cfg["vocab_size"], generator=g, dtype=torch.float64)
    _, grads = O.vjp_sequence(tokens, cfg, wt, dlogits)
    rng = np.random.default_rng(0)
    for name in ("wq", "w2", "rms_ffn_weight", "wcls", "token_embedding_table", "wv"):
        dirn = torch.from_numpy(rng.standard_normal(tuple(wt[name].shape)))
        eps = 1e-6
        wp = dict(wt); wp[name] = wt[name] + eps * dirn
        wm = dict(wt); wm[name] = wt[name] - eps * dirn
        fd = ((O.forward_sequence(tokens, cfg, wp) - O.forward_sequence(tokens, cfg, wm)) * dlogits).sum() / (2 * eps)
        an = (grads[name] * dirn).sum()
        assert abs(fd - an) <= 1e-6 * max(1.0, abs(an)), (name, float(fd), float(an))


def test_fp32_vs_fp64_rounding_bound():
    cfg = O.CONFIGS["tiny"]
    w64 = O.make_weights(cfg, 9, torch.float64)
    w32 = O.cast_weights(w64, torch.float32)
    tokens = O.make_tokens(cfg, 2, 16, 1)
    a = O.forward_sequence(tokens, cfg, w64)
    b = O.forward_sequence(tokens, cfg, w32).double()
    assert (a - b).abs().max() <= 1e-5 + 1e-4 * a.abs().max()


def test_token_vjp_against_level0_and_finite_differences():
    """vjp_token (all-input reverse mode of the reference's call shape): its primal equals Level 0, its cotangents of
    x and of a cache row equal central finite differences of Level 0, and wcls gets exactly zero."""
    import numpy as np
    cfg = O.CONFIGS["tiny"]
    w = O.make_weights(cfg, 3, torch.float64, std=0.2, gains_one=False)
    g = torch.Generator().manual_seed(1)
    L, d = cfg["n_layers"], cfg["dim"]
    x = torch.randn(d, generator=g, dtype=torch.float64)
    kc = torch.randn(L, 3, d, generator=g, dtype=torch.float64)
    vc = torch.randn(L, 3, d, generator=g, dtype=torch.float64)
    dh = torch.randn(d, generator=g, dtype=torch.float64)
    hidden, dx, grads, dk, dv = O.vjp_token(x, cfg, w, kc, vc, dh)
    wn = O.to_numpy(w)
    assert np.abs(hidden.numpy() - O.forward_token(x.numpy(), cfg, wn, kc.numpy(), vc.numpy())).max() < 1e-12

    def f(x_, kc_, vc_):
        return float((torch.from_numpy(O.forward_token(x_.numpy(), cfg, wn, kc_.numpy(), vc_.numpy())) * dh).sum())

    eps = 1e-6
    for i in (0, 5, d - 1):
        xp, xm = x.clone(), x.clone()
        xp[i] += eps
        xm[i] -= eps
        assert abs((f(xp, kc, vc) - f(xm, kc, vc)) / (2 * eps) - float(dx[i])) < 1e-7
    for idx in ((0, 0, 3), (1, 2, 7)):
        for cache, grad, which in ((kc, dk, 0), (vc, dv, 1)):
            cp, cm = cache.clone(), cache.clone()
            cp[idx] += eps
            cm[idx] -= eps
            fd = (f(x, cp, vc) - f(x, cm, vc)) if which == 0 else (f(x, kc, cp) - f(x, kc, cm))
            assert abs(fd / (2 * eps) - float(grad[idx])) < 1e-7
    assert float(grads["wcls"].abs().max()) == 0.0


def test_jvp_sequence_against_finite_differences():
    """Forward mode of Level 1 (the harness's `Forward` row) against central differences along the tangent direction."""
    cfg = O.CONFIGS["tiny"]
    w = O.make_weights(cfg, 3, torch.float64, std=0.2, gains_one=False)
    g = torch.Generator().manual_seed(2)
    dw = {k: 0.1 * torch.randn(v.shape, generator=g, dtype=torch.float64) for k, v in w.items()}
    tok = O.make_tokens(cfg, 2, 8, 1)
    primal, tangent = O.jvp_sequence(tok, cfg, w, dw)
    assert torch.allclose(primal, O.forward_sequence(tok, cfg, w))
    eps = 1e-6
    fd = (O.forward_sequence(tok, cfg, {k: v + eps * dw[k] for k, v in w.items()}) -
          O.forward_sequence(tok, cfg, {k: v - eps * dw[k] for k, v in w.items()})) / (2 * eps)
    assert float((fd - tangent).abs().max()) < 1e-6 * float(tangent.abs().max())


def test_jvp_token_is_the_transpose_of_vjp_token():
    """<d_hidden, J v> == <J^T d_hidden, v> for the all-input tangent v: forward and reverse mode of the reference's
    call shape agree (both were checked against finite differences of Level 0 / Level 1 separately)."""
    cfg = O.CONFIGS["tiny"]
    w = O.make_weights(cfg, 3, torch.float64, std=0.2, gains_one=False)
    g = torch.Generator().manual_seed(4)
    L, d = cfg["n_layers"], cfg["dim"]
    r = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    x, kc, vc, dh = r(d), r(L, 3, d), r(L, 3, d), r(d)
    dx, dkc, dvc = r(d), r(L, 3, d), r(L, 3, d)
    dw = {k: 0.1 * r(*v.shape) for k, v in w.items() if k != "token_embedding_table"}
    hidden, tangent = O.jvp_token(x, cfg, w, kc, vc, dx, dw, dkc, dvc)
    h2, gx, gw, gk, gv = O.vjp_token(x, cfg, w, kc, vc, dh)
    assert torch.allclose(hidden, h2)
    lhs = float((dh * tangent).sum())
    rhs = float((gx * dx).sum() + (gk * dkc).sum() + (gv * dvc).sum() + sum((gw[k] * dw[k]).sum() for k in dw))
    assert abs(lhs - rhs) < 1e-9 * max(1.0, abs(lhs))

"""The reference-shaped Python surface (enzyme_ad.jax) on the GPU: the reference's own call
shape against the golden vector of its forward source, and the jax.vjp-shaped helper."""
import os

import numpy as np
import pytest
import torch

from oracle import llama_ref as O

pytestmark = pytest.mark.gpu


def test_reference_call_shape_against_golden():
    from enzyme_ad.jax import B200Pipeline, enzyme_jax_ir
    gold = np.load(os.path.join(os.path.dirname(__file__), "golden", "llama_golden.npz"))
    cfg = O.CONFIGS["c1"]
    rng = np.random.default_rng(11)
    w = {}
    for name, shape in sorted(O.weight_shapes(cfg).items()):
        w[name] = torch.from_numpy(rng.random(shape).astype(np.float32))
    x = torch.from_numpy(rng.random(cfg["dim"]).astype(np.float32))
    w.pop("token_embedding_table")  # the reference's weight dict has no embedding leaf
    kc = torch.zeros(cfg["n_layers"], 1, cfg["dim"])

    def forward(x, weights, key_cache, value_cache):  # stands for test/llama.py's partial(forward, config)
        raise AssertionError("the body is never traced here")

    fn = enzyme_jax_ir(pipeline_options=B200Pipeline(cfg, torch.float32))(forward)
    out = fn(x, {k: v.cuda() for k, v in w.items()}, kc, kc.clone())
    # uniform[0,1) weights make activations of order 1e2..1e5; the reference's own bar for this test is 1e-3 relative
    np.testing.assert_allclose(out.cpu().numpy(), gold["A_f32"], rtol=1e-3, atol=1e-3)
    np.testing.assert_allclose(out.double().cpu().numpy(), gold["A_f64"], rtol=1e-3, atol=1e-3)


def test_vjp_helper_and_unsupported_entries():
    import enzyme_ad.jax as EJ
    cfg = dict(dim=128, hidden_dim=256, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=512, seq_len=64)
    w = O.make_weights(cfg, 7, torch.float32, std=0.1, gains_one=False)
    tokens = O.make_tokens(cfg, 2, 32, 9)
    dl = torch.randn(2, 32, cfg["vocab_size"], generator=torch.Generator().manual_seed(1))
    ref_logits, ref = O.vjp_sequence(tokens, cfg, {k: v.double() for k, v in w.items()}, dl.double())

    @EJ.enzyme_jax_ir(pipeline_options=EJ.B200Pipeline(cfg, torch.float32))
    def model(tokens, weights):
        raise AssertionError

    wd = {k: v.cuda() for k, v in w.items()}
    logits, pull = EJ.vjp(model, tokens, wd)
    assert torch.allclose(logits.double().cpu(), ref_logits, rtol=1e-4, atol=1e-5)
    no_token_cotangent, grads = pull(dl)
    assert no_token_cotangent is None
    for k, r in ref.items():
        assert float((grads[k].double().cpu() - r).abs().max() / r.abs().max()) < 1e-4, k
    with pytest.raises(NotImplementedError):
        EJ.cpp_call()
    with pytest.raises(NotImplementedError):
        EJ.enzyme_jax_ir(pipeline_options=EJ.JaXPipeline("inline"))(lambda x: x)


def test_harness_rows_and_csv(tmp_path, monkeypatch):
    """The reference-format timing harness: Primal and the three reverse keys, 5-column CSV named after the class."""
    import csv
    import enzyme_ad.jax as EJ
    from enzyme_ad.jax.harness import CSV_HEADER, Llama
    cfg = dict(dim=128, hidden_dim=256, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=512, seq_len=64)
    w = {k: v.cuda() for k, v in O.make_weights(cfg, 7, torch.bfloat16, std=0.1, gains_one=False).items()}
    tokens = O.make_tokens(cfg, 2, 32, 9)
    dl = torch.randn(2, 32, cfg["vocab_size"], generator=torch.Generator().manual_seed(1))

    @EJ.enzyme_jax_ir(pipeline_options=EJ.B200Pipeline(cfg, torch.bfloat16))
    def model(tokens, weights):
        raise AssertionError

    h = Llama(repeat=5, warmup=1)
    h.revprimal = True
    ref_logits, ref = O.vjp_sequence(tokens, cfg, {k: v.double().cpu() for k, v in w.items()}, dl.double())
    # bf16 model against the fp64 oracle on the same bf16 weights: 2e-2 of the largest logit
    h.atol, h.rtol = 2e-2 * float(ref_logits.abs().max()), 2e-2
    dw = {"wq": 0.1 * torch.randn(w["wq"].shape, generator=torch.Generator().manual_seed(2))}
    _, ref_tan = O.jvp_sequence(tokens, cfg, {k: v.double().cpu() for k, v in w.items()}, {k: v.double() for k, v in dw.items()})
    times = h.harness("llama", model, (tokens, w), dl, dins=dw, baseline_primal=ref_logits)
    assert list(times) == ["Primal", "Forward", "PreRev", "PostRev", "BothRev"]
    assert ref_tan.shape == ref_logits.shape
    assert all(0 < t < 1 for t in times.values())
    assert times["BothRev"] > times["Primal"]  # reverse rows include the primal (revprimal)
    monkeypatch.setenv("TEST_UNDECLARED_OUTPUTS_DIR", str(tmp_path))
    path = h.write_results_csv()
    assert os.path.basename(path) == "results_Llama.csv"
    rows = list(csv.reader(open(path)))
    assert rows[0] == CSV_HEADER and len(rows) == 6
    assert [r[3] for r in rows[1:]] == ["Primal", "Forward", "PreRev", "PostRev", "BothRev"]
    assert all(r[:3] == ["llama", "B200", "gpu"] and float(r[4]) > 0 for r in rows[1:])


@pytest.mark.parametrize("pos,zero_cache", [(1, True), (5, False), (0, False)])
def test_token_vjp_all_inputs_matches_oracle(pos, zero_cache):
    """The reference's differentiated call (test/llama.py:315-317): gradients with respect to x, every weight leaf and
    both caches, at the shipped shape (config 1, a one-row zero cache) and with a random 5-row cache."""
    import b200_llama as B
    cfg = O.CONFIGS["c1"]
    L, d = cfg["n_layers"], cfg["dim"]
    w = O.make_weights(cfg, 13, torch.float32, std=0.05, gains_one=False)
    g = torch.Generator().manual_seed(14)
    x = torch.randn(d, generator=g)
    kc = torch.zeros(L, pos, d) if zero_cache else torch.randn(L, pos, d, generator=g)
    vc = torch.zeros(L, pos, d) if zero_cache else torch.randn(L, pos, d, generator=g)
    dh = torch.randn(d, generator=g)
    hidden, dx, grads, dk, dv = O.vjp_token(x.double(), cfg, {k: v.double() for k, v in w.items()}, kc.double(),
                                            vc.double(), dh.double())
    p = B.Plan(cfg, torch.float32)
    p.pack_weights({k: v.cuda().contiguous() for k, v in w.items()}, with_transposed=True)
    got_h, got_dx, packed, got_dk, got_dv = p.token_vjp(x, kc, vc, dh)
    torch.cuda.synchronize()
    assert B.device_status() == 0

    def close(a, b, what):
        scale = float(b.abs().max().clamp_min(1e-30))
        err = float((a.double().cpu() - b).abs().max()) / scale
        assert err < 1e-4, (what, err)

    close(got_h, hidden, "hidden")
    close(got_dx, dx, "dx")
    if pos:
        close(got_dk, dk, "d key_cache")
        close(got_dv, dv, "d value_cache")
    leaves = p.unpack_grads(packed)
    for k, r in grads.items():
        if k == "wcls":
            assert float(leaves[k].abs().max()) == 0.0   # a dead argument: identically zero
        else:
            close(leaves[k], r, k)
    assert float(leaves["token_embedding_table"].abs().max()) == 0.0
    p.close()


def test_harness_reference_call_all_input_gradients_checked_against_oracle(tmp_path, monkeypatch):
    """The reference's test end to end: fn(x, weights, key_cache, value_cache) with pos = 1 zero caches, Primal and the
    three reverse rows, gradients with respect to all four inputs, results checked leaf by leaf (recursive_check) at
    the reference's own tolerance (atol = rtol = 1e-3, test/llama.py:318-319); a wrong baseline must be caught."""
    import enzyme_ad.jax as EJ
    from enzyme_ad.jax.harness import Llama, recursive_check
    cfg = O.CONFIGS["c1"]
    L, d = cfg["n_layers"], cfg["dim"]
    w = O.make_weights(cfg, 17, torch.float32, std=0.05, gains_one=False)
    w.pop("token_embedding_table")
    g = torch.Generator().manual_seed(18)
    x, dx = torch.randn(d, generator=g), torch.randn(d, generator=g)
    kc, vc = torch.zeros(L, 1, d), torch.zeros(L, 1, d)

    @EJ.enzyme_jax_ir(pipeline_options=EJ.B200Pipeline(cfg, torch.float32))
    def forward(x, weights, key_cache, value_cache):
        raise AssertionError("the body is never traced here")

    wfull = dict(w, token_embedding_table=torch.zeros(cfg["vocab_size"], d))
    hidden, rdx, rgrads, rdk, rdv = O.vjp_token(x.double(), cfg, {k: v.double() for k, v in wfull.items()}, kc.double(),
                                                vc.double(), dx.double())
    wd = {k: v.cuda() for k, v in w.items()}
    h = Llama(repeat=3, warmup=1)
    assert h.revprimal is False and h.atol == 1e-3   # the reference's settings for this test
    gt = torch.Generator().manual_seed(19)
    dins = (torch.randn(d, generator=gt), {k: 0.05 * torch.randn(v.shape, generator=gt) for k, v in w.items()},
            torch.randn(L, 1, d, generator=gt), torch.randn(L, 1, d, generator=gt))
    _, ref_tan = O.jvp_token(x.double(), cfg, {k: v.double() for k, v in wfull.items()}, kc.double(), vc.double(),
                             dins[0].double(), {k: v.double() for k, v in dins[1].items()}, dins[2].double(),
                             dins[3].double())
    times = h.harness("llama", forward, (x, wd, kc, vc), dx, dins=dins, baseline_primal=hidden,
                      baseline_tangent=ref_tan, baseline_grads=(rdx, {k: rgrads[k] for k in wd}, rdk, rdv))
    assert list(times) == ["Primal", "Forward", "PreRev", "PostRev", "BothRev"]
    bad = hidden.clone()
    bad[3] += 1.0
    with pytest.raises(AssertionError):
        recursive_check(h, forward(x, wd, kc, vc), bad, "Primal")
    # a function that cannot take the call, or a weight dict that is not llama's, is refused
    @EJ.enzyme_jax_ir(pipeline_options=EJ.B200Pipeline(cfg, torch.float32))
    def two_args(a, b):
        raise AssertionError
    with pytest.raises(TypeError):
        two_args(x, wd, kc, vc)
    with pytest.raises(ValueError):
        forward(x, dict(wd, extra_leaf=torch.zeros(1)), kc, vc)
    with pytest.raises(ValueError):
        forward(x, {k: v for k, v in wd.items() if k != "wq"}, kc, vc)
    with pytest.raises(ValueError):
        forward(x, dict(wd, wq=wd["wq"][:, :10]), kc, vc)


@pytest.mark.parametrize("pos", [1, 4])
def test_token_jvp_all_inputs_matches_oracle(pos):
    """jax.jvp(fn, ins, dins) of the reference's harness: tangents for x, every weight leaf and both caches, at config
    1; and the forward / reverse pair is consistent: <d_hidden, J v> == <J^T d_hidden, v>."""
    import b200_llama as B
    cfg = O.CONFIGS["c1"]
    L, d = cfg["n_layers"], cfg["dim"]
    w = O.make_weights(cfg, 19, torch.float32, std=0.05, gains_one=False)
    g = torch.Generator().manual_seed(20)
    r = lambda *s: torch.randn(*s, generator=g)
    x, kc, vc = r(d), r(L, pos, d), r(L, pos, d)
    dx, dkc, dvc, dh = r(d), r(L, pos, d), r(L, pos, d), r(d)
    dw = {k: 0.05 * r(*v.shape) for k, v in w.items() if k != "token_embedding_table"}
    dbl = lambda t: t.double()
    hidden, tangent = O.jvp_token(dbl(x), cfg, {k: dbl(v) for k, v in w.items()}, dbl(kc), dbl(vc), dbl(dx),
                                  {k: dbl(v) for k, v in dw.items()}, dbl(dkc), dbl(dvc))
    p = B.Plan(cfg, torch.float32)
    p.pack_weights({k: v.cuda().contiguous() for k, v in w.items()}, with_transposed=True)
    got_h, got_t = p.token_jvp(x, kc, vc, dx, dw, dkc, dvc)
    torch.cuda.synchronize()
    assert B.device_status() == 0
    assert float((got_h.double().cpu() - hidden).abs().max() / hidden.abs().max()) < 1e-4
    assert float((got_t.double().cpu() - tangent).abs().max() / tangent.abs().max()) < 1e-4
    # transpose relation with the reverse mode of the same call
    _, gx, packed, gk, gv = p.token_vjp(x, kc, vc, dh)
    gw = p.unpack_grads(packed)
    lhs = float((dh.double() * got_t.double().cpu()).sum())
    rhs = float((gx.double().cpu() * dx).sum() + (gk.double().cpu() * dkc).sum() + (gv.double().cpu() * dvc).sum() +
                sum((gw[k].double().cpu() * dw[k]).sum() for k in dw))
    assert abs(lhs - rhs) < 1e-3 * max(1.0, abs(lhs))
    p.close()


def test_plan_options_round_trip():
    import b200_llama as B
    cfg = dict(O.CONFIGS["c1"], n_layers=1)
    p = B.Plan(cfg, torch.float32)
    for v in (1, 0):
        p.set_option("tp_pipeline", v)
        assert p.get_option("tp_pipeline") == v
    for call in (lambda: p.set_option("no_such_option", 1), lambda: p.get_option("no_such_option")):
        with pytest.raises(B.B200Error) as e:
            call()
        assert e.value.status == 1
    # a plan on one GPU has nothing to tune
    assert p.tune_tensor_parallel(torch.zeros(1, 8, dtype=torch.int32, device="cuda"))["tp_pipeline"] == 0
    p.close()
